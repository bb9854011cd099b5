#!/usr/bin/env python
"""Per-operator timing against the B200 rooflines (the 16384-token operator sweep and the attention shapes).

    python qwen3-triton_b200/benchmarks/op_bench.py [--ops a,b,...] [--scale 1.0] [--iters 10] [--json out.json]

Every operator is timed with CUDA events on the launching stream after 3 warm-up calls; between timed calls
a 256 MB buffer is overwritten so nothing is served from the 126 MB L2 (the bandwidth-bound inputs are also
larger than L2). Reports achieved GB/s (algorithmic bytes) or TFLOP/s and the fraction of the measured peak
in MEASURED_PEAKS.json when present (else the fallback numbers). `--scale 0.125` shrinks the token count for
profiler captures.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import torch  # noqa: E402

from qwen3_triton import _abi  # noqa: E402
from qwen3_triton.kernels.attention import attention_backward, attention_forward  # noqa: E402
from qwen3_triton.kernels.linear import matmul  # noqa: E402


def peaks():
    path = HERE.parent.parent / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, iters):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / self.iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="all")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    hbm, tf, kind = peaks()
    timer = Timer(a.iters)
    T = max(128, int(16384 * a.scale) // 128 * 128)
    H, I, HQ, HK, D, V = 4096, 12288, 32, 8, 128, 151936
    bf = torch.bfloat16
    dev = "cuda"
    st = _abi.stream
    results = []

    def want(name):
        return a.ops == "all" or name in a.ops.split(",")

    def report(name, ms, bytes_=None, flops=None):
        row = {"op": name, "ms": ms}
        if bytes_ is not None:
            row.update(gbs=bytes_ / ms / 1e6, frac=bytes_ / ms / 1e6 / hbm, bound="hbm", bytes=bytes_)
        if flops is not None:
            row.update(tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tf, bound="tensor", flops=flops)
        results.append(row)
        val = f"{row.get('gbs', 0):8.0f} GB/s" if bytes_ is not None else f"{row.get('tflops', 0):8.1f} TFLOP/s"
        print(f"{name:28s} {ms:9.4f} ms  {val}  {row['frac'] * 100:5.1f}% of {kind} peak", flush=True)

    lib = _abi.lib()
    x = torch.randn(T, H, device=dev).to(bf)
    r = torch.randn(T, H, device=dev).to(bf)
    w = torch.ones(H, device=dev, dtype=bf)
    y, y2, inv = torch.empty_like(x), torch.empty_like(x), torch.empty(T, device=dev)
    dw = torch.empty_like(w)
    ws = _abi.workspace(lib.q3_rmsnorm_bwd_workspace_bytes(T, H), dev)
    if want("rmsnorm_fwd"):
        ms = timer(lambda: _abi.call("q3_rmsnorm_fwd", x.data_ptr(), w.data_ptr(), y.data_ptr(), inv.data_ptr(), T, H, 1e-6, 1, st()))
        report("rmsnorm_fwd", ms, bytes_=2 * T * H * 2)
    if want("rmsnorm_bwd"):
        ms = timer(lambda: _abi.call("q3_rmsnorm_bwd", x.data_ptr(), w.data_ptr(), r.data_ptr(), inv.data_ptr(), y.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), T, H, 1, st()))
        report("rmsnorm_bwd", ms, bytes_=3 * T * H * 2)
    if want("add_rmsnorm_fwd"):
        ms = timer(lambda: _abi.call("q3_add_rmsnorm_fwd", x.data_ptr(), r.data_ptr(), w.data_ptr(), y.data_ptr(), y2.data_ptr(), inv.data_ptr(), T, H, 1e-6, 1, st()))
        report("add_rmsnorm_fwd", ms, bytes_=4 * T * H * 2)
    if want("add_rmsnorm_bwd"):
        ms = timer(lambda: _abi.call("q3_add_rmsnorm_bwd", x.data_ptr(), w.data_ptr(), r.data_ptr(), y2.data_ptr(), inv.data_ptr(), y.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), T, H, 1, st()))
        report("add_rmsnorm_bwd", ms, bytes_=4 * T * H * 2)
    if want("norm_rope_fwd") or want("norm_rope_bwd"):
        S = min(4096, T)
        B = T // S
        pos = torch.arange(S, device=dev).repeat(B, 1).contiguous()
        freq = (1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(dev)
        cos, sin = torch.empty(B, S, D, device=dev, dtype=bf), torch.empty(B, S, D, device=dev, dtype=bf)
        _abi.call("q3_rope_tables", pos.data_ptr(), 1, freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, D, 1, st())
        q, k = torch.randn(T, HQ, D, device=dev).to(bf), torch.randn(T, HK, D, device=dev).to(bf)
        qo, ko = torch.empty_like(q), torch.empty_like(k)
        qi, ki = torch.empty(T * HQ, device=dev), torch.empty(T * HK, device=dev)
        wd, dwd = torch.ones(D, device=dev, dtype=bf), torch.empty(D, device=dev, dtype=bf)
        ws2 = _abi.workspace(lib.q3_norm_rope_bwd_workspace_bytes(T, HQ, D), dev)

        dwq, dwk = torch.empty(D, device=dev, dtype=bf), torch.empty(D, device=dev, dtype=bf)
        dq, dk = torch.empty_like(q), torch.empty_like(k)
        ws3 = _abi.workspace(lib.q3_qk_norm_rope_bwd_workspace_bytes(T, HQ, HK, D), dev)

        def fwd():     # q and k in one launch, as the decoder layer calls it
            _abi.call("q3_qk_norm_rope_fwd", q.data_ptr(), k.data_ptr(), wd.data_ptr(), wd.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                      qo.data_ptr(), ko.data_ptr(), qi.data_ptr(), ki.data_ptr(), T, HQ, HK, D, 1e-6, 1, st())

        def bwd():
            _abi.call("q3_qk_norm_rope_bwd", q.data_ptr(), k.data_ptr(), wd.data_ptr(), wd.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                      qo.data_ptr(), ko.data_ptr(), qi.data_ptr(), ki.data_ptr(), dq.data_ptr(), dk.data_ptr(), dwq.data_ptr(),
                      dwk.data_ptr(), ws3.data_ptr(), ws3.numel(), T, HQ, HK, D, 1, st())
        if want("norm_rope_fwd"):
            report("norm_rope_fwd (q+k)", timer(fwd), bytes_=2 * T * (HQ + HK) * D * 2 + 2 * T * D * 2)
        if want("norm_rope_bwd"):
            report("norm_rope_bwd (q+k)", timer(bwd), bytes_=3 * T * (HQ + HK) * D * 2 + 2 * T * D * 2)
        del q, k, qo, ko, dq, dk
    if want("swiglu_fwd") or want("swiglu_bwd"):
        g, u = torch.randn(T, I, device=dev).to(bf), torch.randn(T, I, device=dev).to(bf)
        o1, o2 = torch.empty_like(g), torch.empty_like(g)
        n = T * I
        if want("swiglu_fwd"):
            report("swiglu_fwd", timer(lambda: _abi.call("q3_swiglu_fwd", g.data_ptr(), u.data_ptr(), o1.data_ptr(), n, 1, st())), bytes_=3 * n * 2)
        if want("swiglu_bwd"):
            dy = torch.randn(T, I, device=dev).to(bf)
            report("swiglu_bwd", timer(lambda: _abi.call("q3_swiglu_bwd", g.data_ptr(), u.data_ptr(), dy.data_ptr(), o1.data_ptr(), o2.data_ptr(), n, 1, st())), bytes_=5 * n * 2)
            del dy
        del g, u, o1, o2
    if want("ce_fwd") or want("ce_bwd"):
        S = min(4096, T)
        B = T // S
        logits = (torch.randn(B, S, V, device=dev) * 2).to(bf)
        labels = torch.randint(0, V, (B, S), device=dev)
        n = B * (S - 1)
        lse, tgt, losses = torch.empty(n, device=dev), torch.empty(n, device=dev), torch.empty(n, device=dev)
        loss, cnt = torch.empty((), device=dev), torch.empty((), device=dev, dtype=torch.int32)
        stat = _abi.status_word(dev)
        if want("ce_fwd"):
            report("ce_fwd (materialised logits)", timer(lambda: _abi.call("q3_ce_fwd", logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), tgt.data_ptr(), losses.data_ptr(), loss.data_ptr(), cnt.data_ptr(), B, S, V, -100, 1, stat.data_ptr(), st())), bytes_=T * V * 2)
        if want("ce_bwd"):
            _abi.call("q3_ce_fwd", logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), tgt.data_ptr(), losses.data_ptr(), loss.data_ptr(), cnt.data_ptr(), B, S, V, -100, 1, stat.data_ptr(), st())
            dl = torch.empty_like(logits)
            up = torch.ones(1, device=dev)
            report("ce_bwd", timer(lambda: _abi.call("q3_ce_grad", logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), cnt.data_ptr(), up.data_ptr(), dl.data_ptr(), B * S, B * S, S, V, 0, V, -100, 1, st())), bytes_=2 * T * V * 2)
            del dl
        del logits
    if want("adamw"):
        # Qwen3-8B tensor shapes, as many whole layers as `scale` of 8.19e9 parameters allows
        per_layer = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (12288, 4096), (12288, 4096), (4096, 12288), (4096,), (4096,), (128,), (128,)]
        nlayers = max(1, int(36 * a.scale * 0.5))   # p, g, m, v at full scale would need 131 GB
        shapes = per_layer * nlayers
        from qwen3_triton.runtime.adamw import TritonAdamW
        params = [torch.nn.Parameter(torch.randn(*s, device=dev) * 0.02) for s in shapes]
        for p in params:
            p.grad = torch.randn_like(p) * 1e-3
        opt = TritonAdamW(params, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
        opt.step()
        total = sum(p.numel() for p in params)
        report(f"adamw ({total / 1e9:.2f}e9 params)", timer(opt.step), bytes_=28 * total)
        del params, opt
    if want("adamw_mp"):
        # same tensors, mixed-precision form: bf16 gradient in, fp32 master/moments updated, bf16 copy out
        per_layer = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (12288, 4096), (12288, 4096), (4096, 12288), (4096,), (4096,), (128,), (128,)]
        shapes = per_layer * max(1, int(36 * a.scale * 0.5))
        from qwen3_triton.runtime.adamw import TritonAdamW
        params = [torch.nn.Parameter(torch.randn(*s, device=dev) * 0.02) for s in shapes]
        for p in params:
            p.q3_lowp_grad = (torch.randn_like(p) * 1e-3).to(bf)
            p.q3_lowp_copy = torch.empty_like(p, dtype=bf)
        opt = TritonAdamW(params, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
        opt.step()
        total = sum(p.numel() for p in params)
        report(f"adamw_mp ({total / 1e9:.2f}e9 params)", timer(opt.step), bytes_=28 * total)
        del params, opt
    if want("pack"):
        # one Qwen3-8B decoder layer as an FSDP unit over 8 ranks: shard copy-in, gathered split, gradient chunk-cat
        from qwen3_triton.runtime import ops as pack
        world = 8
        shapes = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (12288, 4096), (12288, 4096), (4096, 12288), (4096,), (4096,), (128,), (128,)]
        numels = [s[0] // world * (s[1] if len(s) > 1 else 1) for s in shapes]
        total = sum(numels)
        shards = [torch.randn(n, device=dev) for n in numels]
        gathered = torch.empty(world * total, device=dev, dtype=bf)
        report("pack copy_in (kernel)", timer(lambda: pack.all_gather_copy_in(shards, gathered, numels, total, 3)), bytes_=6 * total)
        dsts = list(torch.split(gathered.narrow(0, 3 * total, total), numels))
        report("pack copy_in (aten)", timer(lambda: torch._foreach_copy_(dsts, shards)), bytes_=6 * total)
        outs = [torch.empty(world, n, device=dev, dtype=bf) for n in numels]
        g2 = gathered.view(world, -1)
        report("pack split (kernel)", timer(lambda: pack.split_with_sizes_copy(g2, numels, dim=1, out=outs)), bytes_=4 * world * total)
        report("pack split (aten)", timer(lambda: torch.split_with_sizes_copy(g2, numels, dim=1, out=outs)), bytes_=4 * world * total)
        grads = [torch.randn(s, device=dev).to(bf) for s in shapes]
        rs_in = torch.empty(world, total, device=dev)
        report("pack chunk_cat (kernel)", timer(lambda: pack.chunk_cat(grads, 0, world, rs_in)), bytes_=6 * world * total)
        report("pack chunk_cat (aten)", timer(lambda: torch._chunk_cat(grads, 0, world, out=rs_in)), bytes_=6 * world * total)
        del shards, gathered, outs, grads, rs_in
    for name, (M, N, K) in {"gemm_q_fwd": (T, 4096, 4096), "gemm_gate_fwd": (T, 12288, 4096), "gemm_down_fwd": (T, 4096, 12288),
                            "gemm_lm_head_fwd": (T, V, 4096)}.items():
        if want(name) or want("gemm"):
            A, Bm = torch.randn(M, K, device=dev).to(bf), (torch.randn(N, K, device=dev) * 0.02).to(bf)
            report(name, timer(lambda: matmul(A, Bm.t())), flops=2.0 * M * N * K)
            if name == "gemm_q_fwd":
                dy = torch.randn(M, N, device=dev).to(bf)
                report("gemm_q_dgrad", timer(lambda: matmul(dy, Bm)), flops=2.0 * M * N * K)
                report("gemm_q_wgrad", timer(lambda: matmul(dy.t(), A)), flops=2.0 * M * N * K)
            del A, Bm
    if want("step_gemm_vs_library"):
        # The step's GEMM shapes at 2048 tokens per GPU in the three layouts of a linear layer, this library's kernel
        # beside the vendor library's (torch.matmul -> cuBLASLt) on the same tensors: what part of the distance to the
        # peak belongs to the shapes (16 row tiles, 1.73-wave schedules) and what part to the kernel.
        tok = 2048
        for label, n, k in (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate|up", 24576, 4096), ("down", 4096, 12288)):
            xa = torch.randn(tok, k, device=dev).to(bf)
            wa = (torch.randn(n, k, device=dev) * 0.02).to(bf)
            dya = torch.randn(tok, n, device=dev).to(bf)
            fl = 2.0 * tok * n * k
            for form, ours, theirs in (("fwd  X W^T", lambda: matmul(xa, wa.t()), lambda: torch.matmul(xa, wa.t())),
                                       ("dgrad dY W", lambda: matmul(dya, wa), lambda: torch.matmul(dya, wa)),
                                       ("wgrad dY^T X", lambda: matmul(dya.t(), xa), lambda: torch.matmul(dya.t(), xa))):
                report("%s %s (this library)" % (label, form), timer(ours), flops=fl)
                report("%s %s (cuBLASLt)" % (label, form), timer(theirs), flops=fl)
            del xa, wa, dya
    if want("linear_ce"):
        from qwen3_triton.kernels.fused_loss import fused_linear_cross_entropy
        S = min(4096, T)
        B = T // S
        hid = torch.randn(B, S, H, device=dev).to(bf).requires_grad_(True)
        wh = (torch.randn(V, H, device=dev) * 0.02).to(bf).requires_grad_(True)
        lab = torch.randint(0, V, (B, S), device=dev)
        report("linear_ce_fwd (no logits)", timer(lambda: fused_linear_cross_entropy(hid, wh, lab)), flops=2.0 * T * H * V)

        def fb():
            hid.grad = wh.grad = None
            fused_linear_cross_entropy(hid, wh, lab).backward()
        report("linear_ce_fwd+bwd (no logits)", timer(fb), flops=8.0 * T * H * V)
        del hid, wh
    for (B, S) in [(4, 4096), (8, 2048), (2, 8192), (1, 2048)]:
        name = f"attn_B{B}_S{S}"
        if want("attn") or want(name):
            S2 = max(256, int(S * min(1.0, a.scale * 4)) // 128 * 128) if a.scale < 0.25 else S
            q = torch.randn(B, HQ, S2, D, device=dev).to(bf)
            k, v = torch.randn(B, HK, S2, D, device=dev).to(bf), torch.randn(B, HK, S2, D, device=dev).to(bf)
            do = torch.randn_like(q)
            fl = 2.0 * B * HQ * S2 * S2 * D
            out, lse = attention_forward(q, k, v, D ** -0.5)
            report(name + "_fwd", timer(lambda: attention_forward(q, k, v, D ** -0.5)), flops=fl)
            report(name + "_bwd", timer(lambda: attention_backward(q, k, v, out, do, lse, D ** -0.5)), flops=2.5 * fl)
            del q, k, v, do, out
    if want("decode"):
        # decode-time operators at batch 8, 8192 cached tokens: all bound by the bytes they must read once
        from qwen3_triton.inference import kernels as IK
        Bd, Td = 8, 8192
        ck, cv = torch.randn(Bd, HK, Td, D, device=dev).to(bf), torch.randn(Bd, HK, Td, D, device=dev).to(bf)
        qd = torch.randn(Bd, 1, HQ, D, device=dev).to(bf)
        report("decode attention (B8, 8192 keys)", timer(lambda: IK.attention(qd, ck, cv, Td - 1)), bytes_=2 * Bd * HK * Td * D * 2)
        kn, vn = torch.randn(Bd, 1, HK, D, device=dev).to(bf), torch.randn(Bd, 1, HK, D, device=dev).to(bf)
        report("decode cache append", timer(lambda: IK.append(kn, vn, ck, cv, Td - 1)), bytes_=4 * Bd * HK * D * 2)
        xw, wg_ = torch.randn(Bd, H, device=dev).to(bf), (torch.randn(I, H, device=dev) * 0.02).to(bf)
        report("decode gemv 8 x 12288 x 4096", timer(lambda: IK.linear(xw, wg_)), bytes_=I * H * 2)
        wv_ = (torch.randn(V, H, device=dev) * 0.02).to(bf)
        report("decode gemv 8 x 151936 x 4096", timer(lambda: IK.linear(xw, wv_)), bytes_=V * H * 2)
        lg = torch.randn(Bd, V, device=dev).to(bf)
        ids_ = torch.zeros(Bd, 4, dtype=torch.int64, device=dev)
        nx, dn = torch.zeros(Bd, 1, dtype=torch.int64, device=dev), torch.zeros(Bd, dtype=torch.bool, device=dev)
        report("decode select (8 x 151936)", timer(lambda: IK.select(lg, ids_, nx, dn, 1, (151645,), 0)), bytes_=Bd * V * 2)
        del ck, cv, wg_, wv_, lg
    assert _abi.read_status() == 0
    if a.json:
        Path(a.json).write_text(json.dumps({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "kind": kind}, "T": T, "results": results}, indent=1))


if __name__ == "__main__":
    main()
