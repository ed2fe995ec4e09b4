#!/usr/bin/env python
"""Benchmark: DeBERTa-v3-base encoder forward (random-init, synthetic token ids), bf16, batch 8 x seq 2048 per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0).  `value` = tokens/s of the whole job with the batch resident in HBM; `e2e` = the same
through the public model call with the token ids copied from pinned host memory and the last hidden state copied back
every step; `roofline` = the fused attention kernel against the measured dense-bf16 tensor peak, its time taken live
with CUDA events around every attention call of the timed steps; `cpu_baseline` = transformers' eager DeBERTa (the
path the reference falls back to) in fp32 on this box's host cores, on one sequence of the same length.

`--impl reference` times only that CPU path (the reference has no CPU kernel of its own: its flash path needs a GPU and
Triton, and its eager path is transformers').
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

SEQ_LEN = 2048
BATCH_PER_GPU = 8
METRIC = "deberta_v3_base_encoder_tokens_per_s"
WORKLOAD = "DeBERTa-v3-base encoder fwd, random-init, 12 layers, hidden 768, 12 heads, batch 8 x seq 2048 per GPU, mask all ones"


def v3_base_config(backend: str):
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    cfg = DebertaV2Config(
        vocab_size=128100, hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072,
        hidden_act="gelu", hidden_dropout_prob=0.1, attention_probs_dropout_prob=0.1, max_position_embeddings=512,
        type_vocab_size=0, layer_norm_eps=1e-7, relative_attention=True, max_relative_positions=-1,
        position_buckets=256, norm_rel_ebd="layer_norm", share_att_key=True, pos_att_type="c2p|p2c",
        position_biased_input=False, pad_token_id=0)
    cfg.attn_backend = backend
    return cfg


def attn_flops(lengths, heads, head_dim=64, span=256, c2p=True, p2c=True):
    """Algorithmic FLOPs of one attention layer: per sequence and head 4*l^2*D (QK^T and PV) plus 2*l*2S*D per position
    term, valid tokens only; softmax, gathers and in-kernel recomputation are not counted."""
    f = 0
    for n in lengths:
        f += heads * (4 * n * n * head_dim + (int(c2p) + int(p2c)) * 2 * n * 2 * span * head_dim)
    return f


def encoder_linear_flops(tokens, hidden, ffn, layers):
    return layers * 2 * tokens * (4 * hidden * hidden + 2 * hidden * ffn)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]), "measured (MEASURED_PEAKS.json, sustained)"
    return 1400.0, "fallback (1.4 PFLOP/s sustained on this pool)"


class ClockSampler:
    """nvidia-smi in the background during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: transformers' eager encoder, fp32, host cores
# ---------------------------------------------------------------------------------------------------------------------
def cpu_eager_run(steps: int, warmup: int, budget_s: float):
    """Full 12-layer encoder on ONE sequence of SEQ_LEN tokens per step (the eager path holds a B*H*L^2 fp32 score tensor,
    so the 8-sequence batch is sampled by one of its sequences).  Returns (tokens/s, ms/step, steps timed, threads)."""
    from flashdeberta_b200.model import FlashDebertaV2Model
    # every host core this process may run on (torchrun sets OMP_NUM_THREADS=1 for its children, which would leave the
    # baseline single-threaded)
    try:
        usable = len(os.sched_getaffinity(0))
    except AttributeError:
        usable = os.cpu_count() or 1
    torch.set_num_threads(max(1, usable))
    threads = torch.get_num_threads()
    torch.manual_seed(1)
    model = FlashDebertaV2Model(v3_base_config("eager")).eval()
    g = torch.Generator(device="cpu").manual_seed(1)
    ids = torch.randint(1, 128100, (1, SEQ_LEN), generator=g)
    mask = torch.ones(1, SEQ_LEN)
    times = []
    with torch.no_grad():
        t0 = time.perf_counter()
        model(input_ids=ids, attention_mask=mask)
        first = time.perf_counter() - t0
        w_left = max(0, warmup - 1)
        if first * (w_left + steps) > budget_s:  # keep the whole arm within its time budget
            w_left = min(w_left, 1)
            steps = max(1, min(steps, int((budget_s - first * (1 + w_left)) / max(first, 1e-3))))
        for _ in range(w_left):
            model(input_ids=ids, attention_mask=mask)
        for _ in range(steps):
            t0 = time.perf_counter()
            model(input_ids=ids, attention_mask=mask)
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    return SEQ_LEN / (ms / 1e3), ms, len(times), threads


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, ms, steps, threads = cpu_eager_run(args.steps, args.warmup, budget_s=150.0)
    sample = f"1 sequence x {SEQ_LEN} tokens through the full 12-layer fp32 eager encoder per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "reference", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------------------
def gpu_arm(args):
    import torch.distributed as dist
    from flashdeberta_b200 import ops
    from flashdeberta_b200.model import FlashDebertaV2Model

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    torch.manual_seed(1)  # same weights on every rank
    model = FlashDebertaV2Model(v3_base_config("b200")).eval().to(dev).to(torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    B, L = BATCH_PER_GPU, SEQ_LEN
    ids_host = torch.randint(1, 128100, (B, L), generator=g).pin_memory()
    mask_host = torch.ones(B, L, dtype=torch.long).pin_memory()
    ids_dev, mask_dev = ids_host.to(dev), mask_host.to(dev)
    out_host = torch.empty(B, L, 768, dtype=torch.bfloat16).pin_memory()
    tokens_per_step = B * L * world

    def step_resident():
        return model(input_ids=ids_dev, attention_mask=mask_dev).last_hidden_state

    copy_stream = torch.cuda.Stream(device=dev)

    def step_e2e():
        # ids and mask come from pinned host memory, the result goes back to pinned host memory on a second stream, so the
        # device-to-host copy of one step runs beside the next step's kernels (the last copy is waited for before the clock
        # stops, see `timed`)
        ids = ids_host.to(dev, non_blocking=True)
        # the mask is handed over where it is, in pinned host memory: the model reads the lengths there and copies it to
        # the device itself (the bytes are counted in h2d_bytes_per_step)
        out = model(input_ids=ids, attention_mask=mask_host).last_hidden_state
        done = torch.cuda.Event()
        done.record()
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done)
            out_host.copy_(out, non_blocking=True)
        out.record_stream(copy_stream)
        return out

    def timed(fn, steps, log_attention=False):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if log_attention:
            ops.event_log = []
        t0.record()
        for _ in range(steps):
            fn()
        torch.cuda.current_stream().wait_stream(copy_stream)  # the last result has reached the host
        t1.record()
        barrier()
        ms = t0.elapsed_time(t1)
        attn_ms = None
        if log_attention:
            attn_ms = [a.elapsed_time(b) for a, b in ops.event_log]
            ops.event_log = None
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms, attn_ms

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step_resident()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = ops.launch_count()
        ms_total, attn_ms = timed(step_resident, args.steps, log_attention=True)
        launches = ops.launch_count() - l0
        for _ in range(2):
            step_e2e()
        ms_e2e, _ = timed(step_e2e, args.steps)
        clocks = sampler.stop() if rank == 0 else None
        ops.check_status(dev)

    ms_step = ms_total / args.steps
    value = tokens_per_step / (ms_step / 1e3)
    e2e_value = tokens_per_step / (ms_e2e / args.steps / 1e3)

    # roofline of the fused attention kernel (per launch = one layer's attention on this rank's batch)
    f_launch = attn_flops([L] * B, heads=12)
    attn_avg_ms = sum(attn_ms) / len(attn_ms)
    achieved = f_launch / (attn_avg_ms / 1e3) / 1e12
    peak, peak_src = measured_peaks()
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "attn_fwd_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f).get("dram_bytes_per_launch")
    total_flops = 12 * f_launch + encoder_linear_flops(B * L, 768, 3072, 12)

    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": B * world, "seq_len": L, "parallelism": f"dp{world}",
                   "l2": "per-step working set (weights + activations, > 1 GB) exceeds the 126 MB L2; no explicit flush"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": ids_host.numel() * 8 + mask_host.numel() * 8,
                "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"kernel": "attn_fwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                     "launch_ms": attn_avg_ms, "flops_per_launch": f_launch,
                     "note": "events bracket one fdb_attn_fwd call (the fused kernel; its two set-up kernels run only while a module's workspace is not prepared)"},
        "attention_share_of_step": attn_avg_ms * 12 / ms_step,
        "model_tflops": total_flops / (ms_step / 1e3) / 1e12,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            tps, ms, steps, threads = cpu_eager_run(2, 1, budget_s=40.0)
            line["cpu_baseline"] = {
                "value": tps, "unit": "tokens/s", "cores": threads, "kind": "reference", "host_cpus": os.cpu_count(),
                "sample": f"1 sequence x {SEQ_LEN} tokens, full 12-layer fp32 eager encoder (transformers), {steps} step(s)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def varlen_run(args):
    """Extra measurement (not the headline line): the packed-batch configuration — DeBERTa-v3-large encoder, 256 sequences
    with log-uniform lengths in [64, 8192] (seed 2, 350907 tokens), bf16, sharded across the ranks by token count with
    one final gather.  Prints one JSON line with "config": {"workload": "varlen ..."}."""
    import torch.distributed as dist
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    from flashdeberta_b200 import ops
    from flashdeberta_b200.dist import partition_by_tokens
    from flashdeberta_b200.model import FlashDebertaV2Model

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = DebertaV2Config(
        vocab_size=128100, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096,
        hidden_act="gelu", max_position_embeddings=512, type_vocab_size=0, layer_norm_eps=1e-7, relative_attention=True,
        max_relative_positions=-1, position_buckets=256, norm_rel_ebd="layer_norm", share_att_key=True,
        pos_att_type="c2p|p2c", position_biased_input=False, pad_token_id=0)
    cfg.attn_backend = "b200"
    torch.manual_seed(2)
    model = FlashDebertaV2Model(cfg).eval().to(dev).to(torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(2)
    u = torch.rand(256, dtype=torch.float64, generator=g)
    lens = torch.floor(torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))).long().tolist()
    mine = partition_by_tokens(lens, world)[rank]
    Lr = max(lens[i] for i in mine)
    ids = torch.zeros(len(mine), Lr, dtype=torch.long)
    mask = torch.zeros(len(mine), Lr, dtype=torch.long)
    for row, i in enumerate(mine):
        ids[row, : lens[i]] = torch.randint(1, 128100, (lens[i],), generator=g)
        mask[row, : lens[i]] = 1
    ids, mask = ids.to(dev), mask.to(dev)
    my_tokens = sum(lens[i] for i in mine)

    def step():
        return model(input_ids=ids, attention_mask=mask).last_hidden_state

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            step()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ops.event_log = []
        t0.record()
        for _ in range(args.steps):
            out = step()
        t1.record()
        barrier()
        ms = t0.elapsed_time(t1)
        attn_ms = sum(a.elapsed_time(b) for a, b in ops.event_log)  # rank 0's own fused-attention calls
        ops.event_log = None
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        ops.check_status(dev)
    total = sum(lens)
    if rank == 0:
        f_attn = 24 * attn_flops(lens, heads=16)
        f_lin = encoder_linear_flops(total, 1024, 4096, 24)
        print(json.dumps({
            "metric": "deberta_v3_large_encoder_tokens_per_s", "value": total / (ms / args.steps / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "ms_per_step": ms / args.steps, "scaling": "strong", "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "varlen packed batch, DeBERTa-v3-large encoder, 256 sequences, lengths log-uniform in "
                                   "[64, 8192] (seed 2)", "total_tokens": total, "tokens_rank0": my_tokens,
                       "parallelism": f"dp{world}, sequences split by token count"},
            "model_tflops": (f_attn + f_lin) / (ms / args.steps / 1e3) / 1e12,
            "attention_share_of_step": attn_ms / ms,
            "attention_tflops_rank0": 24 * attn_flops([lens[i] for i in mine], heads=16) * args.steps / (attn_ms / 1e3) / 1e12,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def fp8_run(args):
    """Extra measurement (not the headline line): the e4m3 configuration — DeBERTa-v3-large encoder, random-init, attention
    operands quantised to e4m3 with per-(sequence, head) scales (`config.attn_fp8`), linears in bf16; 8 sequences of 4096
    tokens per GPU (the per-GPU share of the 64-sequence batch at 8 GPUs; weak scaling), ids uniform from seed 4.  Also times
    the bf16 attention on the same model and inputs.  Prints one JSON line with "config": {"workload": "fp8 ..."}."""
    import torch.distributed as dist
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    from flashdeberta_b200 import ops
    from flashdeberta_b200.model import FlashDebertaV2Model

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, L = 8, 4096

    def build(fp8: bool):
        cfg = DebertaV2Config(
            vocab_size=128100, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096,
            hidden_act="gelu", max_position_embeddings=512, type_vocab_size=0, layer_norm_eps=1e-7,
            relative_attention=True, max_relative_positions=-1, position_buckets=256, norm_rel_ebd="layer_norm",
            share_att_key=True, pos_att_type="c2p|p2c", position_biased_input=False, pad_token_id=0)
        cfg.attn_backend = "b200"
        cfg.attn_fp8 = fp8
        torch.manual_seed(4)
        return FlashDebertaV2Model(cfg).eval().to(dev).to(torch.bfloat16)

    g = torch.Generator(device="cpu").manual_seed(4 + rank)
    ids = torch.randint(1, 128100, (B, L), generator=g).to(dev)
    mask = torch.ones(B, L, dtype=torch.long, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(model):
        with torch.no_grad():
            for _ in range(max(args.warmup, 3)):
                model(input_ids=ids, attention_mask=mask)
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(args.steps):
                out = model(input_ids=ids, attention_mask=mask).last_hidden_state
            t1.record()
            barrier()
            ms = t0.elapsed_time(t1)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
            ops.check_status(dev)
        return ms / args.steps, out

    m8 = build(True)
    ms8, out8 = timed(m8)
    del m8
    m16 = build(False)
    ms16, out16 = timed(m16)
    diff = (out8.float() - out16.float()).abs()
    if rank == 0:
        tokens = B * L * world
        f = 24 * attn_flops([L] * B, heads=16) + encoder_linear_flops(B * L, 1024, 4096, 24)
        print(json.dumps({
            "metric": "deberta_v3_large_encoder_tokens_per_s", "value": tokens / (ms8 / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "ms_per_step": ms8, "scaling": "weak", "dtype": "e4m3 attention, bf16 linears",
            "data": "synthetic",
            "config": {"workload": "fp8: DeBERTa-v3-large encoder, 8 x 4096 tokens per GPU, e4m3 attention operands with "
                                   "per-(sequence, head) scales (seed 4)", "global_batch": B * world, "seq_len": L,
                       "parallelism": f"dp{world}"},
            "bf16_attention_ms_per_step": ms16, "bf16_attention_tokens_per_s": tokens / (ms16 / 1e3),
            "last_hidden_state_vs_bf16_attention": {"max_abs": diff.max().item(), "mean_abs": diff.mean().item()},
            "model_tflops": f / (ms8 / 1e3) / 1e12}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--varlen", action="store_true", help="measure the packed v3-large configuration instead")
    ap.add_argument("--fp8", action="store_true", help="measure the e4m3-attention v3-large configuration instead")
    args = ap.parse_args()
    if args.varlen:
        varlen_run(args)
    elif args.fp8:
        fp8_run(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
