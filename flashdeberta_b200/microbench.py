"""Attention-only microbenchmark of the fused kernel (CUDA events, inputs rotated so consecutive launches do not find
their operands in L2).

    python -m flashdeberta_b200.microbench --batch 8 --seq 2048 --heads 12 [--iters 30] [--no-pos] [--packed-lens 700,130]

Prints one JSON line: median/min ms per launch and algorithmic TFLOP/s (4*l^2*D + 2*l*2S*D per position term, per
sequence and head).

    python -m flashdeberta_b200.microbench --add-layernorm --rows 16384 --hidden 768

times the fused residual + LayerNorm kernel instead (algorithmic bytes: 3 * rows * hidden * 2, four rotated buffers).

    python -m flashdeberta_b200.microbench --linear-gelu --rows 16384 --hidden 768 --out-features 3072

times the fused linear + GELU kernel (2 * rows * hidden * out_features FLOP) beside torch's linear followed by gelu.

    python -m flashdeberta_b200.microbench --reference-triton --batch 8 --seq 2048

times the reference's own attention path on the same GPU and the same q, k, v: the two bias GEMMs of
src/flashdeberta/model.py:189-192 followed by flash_attention_with_disentangled (src/flashdeberta/ops/flash_attention.py:1088,
Triton, compiled by the installed Triton), beside this library's fused call, and reports the largest difference between the
two outputs.  Needs an unmodified copy of the reference package importable as ``flashdeberta`` (looked for under
``baseline/_ref`` next to this package).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from . import ops


def attn_flops(lengths, heads, head_dim=64, span=256, c2p=True, p2c=True):
    return sum(heads * (4 * n * n * head_dim + (int(c2p) + int(p2c)) * 2 * n * 2 * span * head_dim) for n in lengths)


def bench_add_layernorm(rows: int, hidden: int, iters: int, warmup: int, sets: int):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(0)
    xs = [torch.randn(rows, hidden, generator=g).bfloat16().to(dev) for _ in range(sets)]
    rs = [torch.randn(rows, hidden, generator=g).bfloat16().to(dev) for _ in range(sets)]
    w, b = torch.ones(hidden, dtype=torch.bfloat16, device=dev), torch.zeros(hidden, dtype=torch.bfloat16, device=dev)
    for i in range(warmup):
        ops.add_layernorm(xs[i % sets], rs[i % sets], w, b, 1e-7)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.add_layernorm(xs[i % sets], rs[i % sets], w, b, 1e-7)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    nbytes = 3 * rows * hidden * 2
    med, mn = statistics.median(times), min(times)
    print(json.dumps({"op": "add_layernorm", "rows": rows, "hidden": hidden, "ms_median": med, "ms_min": mn,
                      "gbs_median": nbytes / med / 1e6, "gbs_best": nbytes / mn / 1e6, "bytes": nbytes,
                      "l2": f"{sets} buffer sets rotated ({sets * 3 * rows * hidden * 2 >> 20} MiB; the output is allocated per call)"}))


def bench_linear_gelu(rows: int, k: int, n: int, iters: int, warmup: int, sets: int):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(0)
    xs = [torch.randn(rows, k, generator=g).bfloat16().to(dev) for _ in range(sets)]
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(dev)
    b = torch.randn(n, generator=g).bfloat16().to(dev)
    F = torch.nn.functional
    res = {}
    for name, fn in (("fused", lambda x: ops.linear_gelu(x, w, b)), ("torch", lambda x: F.gelu(F.linear(x, w, b)))):
        for i in range(warmup):
            fn(xs[i % sets])
        torch.cuda.synchronize()
        times = []
        for i in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(xs[i % sets])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        res[name] = statistics.median(times)
    ops.check_status()
    flops = 2 * rows * k * n
    print(json.dumps({"op": "linear_gelu", "rows": rows, "in_features": k, "out_features": n, "ms_median": res["fused"],
                      "tflops_median": flops / res["fused"] / 1e9, "torch_linear_then_gelu_ms": res["torch"],
                      "flops": flops, "l2": f"{sets} input buffers rotated; the output is allocated per call"}))


def _time(fn, iters: int, warmup: int):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


def bench_reference_triton(B: int, L: int, H: int, iters: int, warmup: int, nsets: int):
    """The reference's attention path (bias GEMMs + its Triton kernel) beside the fused call, same inputs."""
    ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    try:
        from flashdeberta.ops.flash_attention import flash_attention_with_disentangled
    except Exception as e:  # the copy is not part of this repository's history
        print(json.dumps({"op": "reference_triton", "unavailable": f"cannot import the reference package from {ref_root}: {e!r}"}))
        return
    import triton
    dev = torch.device("cuda")
    D = 64
    g = torch.Generator(device="cpu").manual_seed(0)
    sets = []
    for _ in range(nsets):
        q, k, v = (torch.randn(B, L, H, D, generator=g).bfloat16().to(dev) for _ in range(3))
        # the reference's kernel wants (B, H, L, D) contiguous (its module makes these copies, model.py:137-140; they are
        # left out of its time here)
        sets.append((q, k, v, *(t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))))
    pk, pq = (torch.randn(H, 512, D, generator=g).mul_(0.5).bfloat16().to(dev) for _ in range(2))
    sm_scale = 1.0 / (3 * D) ** 0.5
    kw = dict(max_seqlen=L, position_buckets=256, max_relative_positions=512)

    def ours(i):
        q, k, v = sets[i % nsets][:3]
        return ops.disentangled_attention(q, k, v, pk, pq, **kw)

    def theirs(i):
        qt, kt, vt = sets[i % nsets][3:]
        c2p = torch.matmul(qt, pk.unsqueeze(0).transpose(-1, -2))   # model.py:189-190
        p2c = torch.matmul(kt, pq.unsqueeze(0).transpose(-1, -2))   # model.py:191-192
        return flash_attention_with_disentangled(qt, kt, vt, c2p, p2c, False, sm_scale, 256, 512)

    def theirs_kernel_only(i):
        qt, kt, vt = sets[i % nsets][3:]
        return flash_attention_with_disentangled(qt, kt, vt, bias[0], bias[1], False, sm_scale, 256, 512)

    with torch.no_grad():
        o_ours = ours(0)
        o_ref = theirs(0).permute(0, 2, 1, 3)
        diff = (o_ours.float() - o_ref.float()).abs()
        qt, kt = sets[0][3], sets[0][4]
        bias = (torch.matmul(qt, pk.unsqueeze(0).transpose(-1, -2)), torch.matmul(kt, pq.unsqueeze(0).transpose(-1, -2)))
        ms_ours = _time(ours, iters, warmup)
        ms_ref = _time(theirs, iters, warmup)
        ms_ref_k = _time(theirs_kernel_only, iters, warmup)
    ops.check_status()
    f = attn_flops([L] * B, H)
    print(json.dumps({
        "op": "reference_triton", "batch": B, "seq": L, "heads": H, "triton": triton.__version__,
        "fused_ms_median": ms_ours[0], "fused_tflops": f / ms_ours[0] / 1e9,
        "reference_ms_median": ms_ref[0], "reference_tflops": f / ms_ref[0] / 1e9,
        "reference_kernel_only_ms_median": ms_ref_k[0],
        "speedup": ms_ref[0] / ms_ours[0],
        "max_abs_diff_between_outputs": diff.max().item(), "mean_abs_diff_between_outputs": diff.mean().item(),
        "note": "reference = bias GEMMs (model.py:189-192) + flash_attention_with_disentangled; its (B,H,L,D) copies are not timed"}))


def bench_backward(B: int, L: int, H: int, iters: int, warmup: int, with_reference: bool):
    """Forward + backward of the attention op (gradients of q, k, v and both position tables), and the same through the
    reference's autograd function (its bias GEMMs included, so that the table gradients exist there too) when asked."""
    dev = torch.device("cuda")
    D = 64
    g = torch.Generator(device="cpu").manual_seed(0)
    q, k, v, do = (torch.randn(B, L, H, D, generator=g).bfloat16().to(dev) for _ in range(4))
    pk, pq = (torch.randn(H, 512, D, generator=g).mul_(0.5).bfloat16().to(dev) for _ in range(2))
    kw = dict(max_seqlen=L, position_buckets=256, max_relative_positions=512)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, pk, pq)]

    def ours(i):
        out = ops.disentangled_attention(*leaves, **kw)
        return torch.autograd.grad(out, leaves, do)

    def ours_fwd(i):
        with torch.no_grad():
            return ops.disentangled_attention(q, k, v, pk, pq, **kw)

    g_ours = ours(0)
    ms = _time(ours, iters, warmup)
    ms_f = _time(ours_fwd, iters, warmup)
    ops.check_status()
    f = attn_flops([L] * B, H)
    line = {"op": "attention_fwd_bwd", "batch": B, "seq": L, "heads": H, "fwd_bwd_ms_median": ms[0],
            "fwd_ms_median": ms_f[0], "bwd_ms": ms[0] - ms_f[0],
            "bwd_tflops_at_2.5x_fwd_flops": 2.5 * f / max(ms[0] - ms_f[0], 1e-9) / 1e9}
    if with_reference:
        ref_root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        try:
            from flashdeberta.ops.flash_attention import flash_attention_with_disentangled
            sm_scale = 1.0 / (3 * D) ** 0.5
            rl = [t.detach().clone().requires_grad_(True) for t in
                  (q.permute(0, 2, 1, 3).contiguous(), k.permute(0, 2, 1, 3).contiguous(), v.permute(0, 2, 1, 3).contiguous(), pk, pq)]
            dot = do.permute(0, 2, 1, 3).contiguous()

            def theirs(i):
                c2p = torch.matmul(rl[0], rl[3].unsqueeze(0).transpose(-1, -2))
                p2c = torch.matmul(rl[1], rl[4].unsqueeze(0).transpose(-1, -2))
                out = flash_attention_with_disentangled(rl[0], rl[1], rl[2], c2p, p2c, False, sm_scale, 256, 512)
                return torch.autograd.grad(out, rl, dot)

            g_ref = theirs(0)
            ms_r = _time(theirs, iters, warmup)
            line["reference_fwd_bwd_ms_median"] = ms_r[0]
            line["speedup_fwd_bwd"] = ms_r[0] / ms[0]
            for name, a, b in zip(("dq", "dk", "dv"), g_ours[:3], g_ref[:3]):
                b = b.permute(0, 2, 1, 3)
                line["rel_diff_" + name] = ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()
            for name, a, b in zip(("dpos_key", "dpos_query"), g_ours[3:], g_ref[3:]):
                line["rel_diff_" + name] = ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()
        except Exception as e:  # the copy is not part of this repository's history; its Triton code may not compile here
            line["reference_unavailable"] = repr(e)[:300]
    print(json.dumps(line))


def bench_eager_gpu(B: int, L: int, H: int, iters: int, warmup: int):
    """transformers' eager DisentangledSelfAttention module (the reference's fallback class, src/flashdeberta/model.py:255)
    on the GPU in fp32 and bf16, beside this package's module with the same weights; whole module, projections included."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention

    from .attention import FlashDisentangledSelfAttention

    class Cfg:
        hidden_size = H * 64
        num_attention_heads = H
        attention_probs_dropout_prob = 0.0
        hidden_dropout_prob = 0.0
        pos_att_type = ["c2p", "p2c"]
        relative_attention = True
        position_buckets = 256
        max_relative_positions = 512
        max_position_embeddings = 512
        share_att_key = True

    dev = torch.device("cuda")
    torch.manual_seed(0)
    eager = DisentangledSelfAttention(Cfg()).eval().to(dev)
    flash = FlashDisentangledSelfAttention(Cfg()).eval().to(dev)
    flash.load_state_dict(eager.state_dict())
    flash = flash.to(torch.bfloat16)
    x = torch.randn(B, L, H * 64, device=dev)
    rel = torch.randn(512, H * 64, device=dev) * 0.02
    mask2 = torch.ones(B, L, device=dev)
    mask4 = mask2[:, None, None, :] * mask2[:, None, :, None]
    res = {"op": "eager_gpu", "batch": B, "seq": L, "heads": H}
    f = attn_flops([L] * B, H)
    with torch.no_grad():
        for name, dt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
            m = eager.to(dt)
            xx, rr, mm = x.to(dt), rel.to(dt), mask4.to(dt)
            med, _ = _time(lambda i: m(xx, mm, rel_embeddings=rr), iters, warmup)
            res[f"eager_{name}_ms"] = med
            res[f"eager_{name}_attn_tflops"] = f / med / 1e9
        xb, rb = x.bfloat16(), rel.bfloat16()
        med, _ = _time(lambda i: flash(xb, mask2, rel_embeddings=rb), iters, warmup)
        res["fused_module_bf16_ms"] = med
        res["fused_module_attn_tflops"] = f / med / 1e9
    ops.check_status()
    res["note"] = "whole attention module incl. q/k/v and position projections; TFLOP/s divides the attention FLOPs only"
    print(json.dumps(res))


def bench_packed256(H: int, iters: int, warmup: int, tune: int):
    """The fused attention on the packed benchmark batch: 256 sequences with lengths log-uniform in [64, 8192] (seed 2,
    350907 tokens) behind one cu_seqlens, c2p + p2c, bf16."""
    import math
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(2)
    u = torch.rand(256, dtype=torch.float64, generator=g)
    lens = torch.floor(torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))).long().tolist()
    T, D = sum(lens), 64
    gd = torch.Generator(device=dev).manual_seed(2)
    sets = [tuple(torch.randn(T, H, D, generator=gd, device=dev).bfloat16() for _ in range(3)) for _ in range(2)]
    pk, pq = (torch.randn(H, 512, D, generator=gd, device=dev).mul_(0.5).bfloat16() for _ in range(2))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    kw = dict(cu_seqlens=cu, max_seqlen=max(lens), position_buckets=256, max_relative_positions=512, tune=tune)
    med, mn = _time(lambda i: ops.disentangled_attention(*sets[i % 2], pk, pq, **kw), iters, warmup)
    ops.check_status()
    f = attn_flops(lens, H)
    print(json.dumps({"workload": "packed 256 sequences, 350907 tokens", "heads": H, "ms_median": med, "ms_min": mn,
                      "tflops_median": f / med / 1e9, "flops": f}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--sets", type=int, default=4, help="independent input sets rotated between launches")
    ap.add_argument("--no-pos", action="store_true")
    ap.add_argument("--packed256", action="store_true", help="the packed 256-sequence benchmark batch (use --heads 16)")
    ap.add_argument("--tune", type=int, default=0, help="fdb_attn_params.tune bits (which kernels the call is split into)")
    ap.add_argument("--fp8", action="store_true", help="e4m3 operands (quantised once, outside the timed region)")
    ap.add_argument("--valid", type=int, default=0, help="valid length of every sequence (default: all)")
    ap.add_argument("--add-layernorm", action="store_true", help="time fdb_add_layernorm instead of the attention")
    ap.add_argument("--linear-gelu", action="store_true", help="time fdb_linear_gelu (rows x hidden -> out-features)")
    ap.add_argument("--eager-gpu", action="store_true",
                    help="time transformers' eager attention module on the GPU (fp32, bf16) beside this package's module")
    ap.add_argument("--reference-triton", action="store_true",
                    help="time the reference's bias GEMMs + Triton kernel beside the fused call on the same inputs")
    ap.add_argument("--backward", action="store_true", help="time forward + backward of the attention op")
    ap.add_argument("--out-features", type=int, default=3072)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=768)
    args = ap.parse_args()
    if args.eager_gpu:
        return bench_eager_gpu(args.batch, args.seq, args.heads, args.iters, args.warmup)
    if args.backward:
        return bench_backward(args.batch, args.seq, args.heads, args.iters, args.warmup, args.reference_triton)
    if args.reference_triton:
        return bench_reference_triton(args.batch, args.seq, args.heads, args.iters, args.warmup, args.sets)
    if args.linear_gelu:
        return bench_linear_gelu(args.rows, args.hidden, args.out_features, args.iters, args.warmup, args.sets)
    if args.add_layernorm:
        return bench_add_layernorm(args.rows, args.hidden, args.iters, args.warmup, max(args.sets, 8))
    dev = torch.device("cuda")
    if args.packed256:
        return bench_packed256(args.heads, args.iters, args.warmup, args.tune)
    B, L, H, D = args.batch, args.seq, args.heads, 64
    g = torch.Generator(device="cpu").manual_seed(0)
    sets = []
    for _ in range(args.sets):
        q, k, v = (torch.randn(B, L, H, D, generator=g).bfloat16().to(dev) for _ in range(3))
        sets.append((q, k, v))
    pk = pq = None
    if not args.no_pos:
        pk, pq = (torch.randn(H, 512, D, generator=g).mul_(0.5).bfloat16().to(dev) for _ in range(2))
    lens = [args.valid or L] * B
    kw = dict(max_seqlen=L, position_buckets=256, max_relative_positions=512, tune=args.tune)
    if args.valid:
        kw["seq_lens"] = torch.tensor(lens, dtype=torch.int32, device=dev)
    if args.fp8:
        slabs = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=dev)
        scales = {}
        qsets = []
        for (q, k, v) in sets:
            (q8, sq), (k8, sk), (v8, sv) = (ops.quantize_e4m3(t, slabs) for t in (q, k, v))
            qsets.append((q8, k8, v8))
            scales = {"q_scale": sq, "k_scale": sk, "v_scale": sv}  # same distribution in every set
        sets = qsets
        if pk is not None:
            tslab = torch.arange(0, (H + 1) * 512, 512, dtype=torch.int32, device=dev)
            pk, spk = ops.quantize_e4m3(pk.view(H * 512, 1, D), tslab)
            pq, spq = ops.quantize_e4m3(pq.view(H * 512, 1, D), tslab)
            pk, pq = pk.view(H, 512, D), pq.view(H, 512, D)
            scales.update(pos_key_scale=spk.view(H), pos_query_scale=spq.view(H))
        kw["scales"] = scales
    for i in range(args.warmup):
        ops.disentangled_attention(*sets[i % args.sets], pk, pq, **kw)
    torch.cuda.synchronize()
    times = []
    for i in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.disentangled_attention(*sets[i % args.sets], pk, pq, **kw)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ops.check_status()
    f = attn_flops(lens, H, c2p=not args.no_pos, p2c=not args.no_pos)
    med, mn = statistics.median(times), min(times)
    print(json.dumps({"batch": B, "seq": L, "heads": H, "valid": lens[0], "pos": not args.no_pos, "fp8": args.fp8, "ms_median": med,
                      "ms_min": mn, "tflops_median": f / med / 1e9, "tflops_best": f / mn / 1e9,
                      "flops": f, "l2": f"{args.sets} input sets rotated ({args.sets * 3 * B * L * H * D * 2 >> 20} MiB)"}))


if __name__ == "__main__":
    main()
