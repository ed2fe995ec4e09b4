#!/usr/bin/env python
"""Benchmark: DeBERTa-v3-large encoder forward on a packed batch of 256 sequences (random-init, synthetic token ids),
bf16, strong scaling over the GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

The 256 sequences (lengths log-uniform in [64, 8192] from seed 2, 350907 tokens) are split across the ranks by whole
sequences with a balanced cost (tokens, plus the attention's quadratic term with a weight measured in the warm-up), each
rank runs the fused path on its packed shard, and one all-gather brings the last hidden state together on every rank.
One JSON line on stdout (rank 0):

* `value`   tokens/s of the whole job, token ids resident in HBM, the final gather inside the timed region;
* `e2e`     the same through the public model call with the ids copied from pinned host memory every step and the gathered
            result copied back to pinned host memory on rank 0;
* `roofline` the fused attention (every fdb_attn_fwd call of the timed steps on rank 0, CUDA events on the launching
            stream) against the measured dense-bf16 tensor peak;
* `cpu_baseline` transformers' eager DeBERTa (the path the reference falls back to) in fp32 on this box's host cores, on
            one sequence of the batch;
* `extra`   at one GPU: the DeBERTa-v3-base 8 x 2048 step, the attention alone at 4 x 4096 x 12 heads, and the eager
            attention layer of the CPU-runnable configuration (batch 2 x 512) on the host cores.

`--impl reference` times only the CPU path (the reference has no CPU kernel of its own: its flash path needs a GPU and
Triton, and its eager path is transformers'); it does not import this repository's package.
`--c2` / `--fp8` print the DeBERTa-v3-base 8 x 2048 line / the e4m3-attention v3-large line instead.
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

METRIC = "deberta_v3_large_packed_tokens_per_s"
WORKLOAD = ("DeBERTa-v3-large encoder fwd (24 layers, hidden 1024, 16 heads, FFN 4096), random-init, bf16, one packed batch of "
            "256 sequences with lengths log-uniform in [64, 8192] (seed 2, 350907 tokens), sharded by whole sequences, one "
            "final all-gather")
CPU_SAMPLE_SEQ = 2  # the sequence of the batch the CPU arm runs (1993 tokens)


def deberta_config(size: str, **extra):
    from transformers.models.deberta_v2.configuration_deberta_v2 import DebertaV2Config
    dims = dict(base=(768, 12, 12, 3072), large=(1024, 24, 16, 4096))[size]
    cfg = DebertaV2Config(
        vocab_size=128100, hidden_size=dims[0], num_hidden_layers=dims[1], num_attention_heads=dims[2],
        intermediate_size=dims[3], hidden_act="gelu", hidden_dropout_prob=0.1, attention_probs_dropout_prob=0.1,
        max_position_embeddings=512, type_vocab_size=0, layer_norm_eps=1e-7, relative_attention=True,
        max_relative_positions=-1, position_buckets=256, norm_rel_ebd="layer_norm", share_att_key=True,
        pos_att_type="c2p|p2c", position_biased_input=False, pad_token_id=0)
    for k, v in extra.items():
        setattr(cfg, k, v)
    return cfg


def packed_batch(seed: int = 2):
    """The 256 lengths and the packed token ids of the benchmark batch (CPU tensors, one seeded generator)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    u = torch.rand(256, dtype=torch.float64, generator=g)
    lens = torch.floor(torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))).long().tolist()
    ids = torch.randint(1, 128100, (sum(lens),), generator=g)
    return lens, ids


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
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback (1.59 / 1.4 PFLOP/s on this pool)"}


def usable_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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
# CPU arm: transformers' eager encoder, fp32, host cores.  Imports nothing of this repository's package.
# ---------------------------------------------------------------------------------------------------------------------
def cpu_eager_encoder(steps: int, warmup: int, budget_s: float):
    """The 24-layer eager encoder (transformers' DebertaV2Model, fp32) on ONE sequence of the packed batch per step: eager
    attention holds an H * L^2 fp32 score tensor per layer, so the batch is sampled by one of its sequences.
    Returns (tokens/s, ms/step, steps timed, threads, sequence length)."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Model
    # every host core this process may run on (torchrun sets OMP_NUM_THREADS=1 for its children, which would leave the
    # baseline single-threaded)
    torch.set_num_threads(max(1, usable_cores()))
    threads = torch.get_num_threads()
    torch.manual_seed(2)
    model = DebertaV2Model(deberta_config("large")).eval()
    lens, ids = packed_batch()
    start = sum(lens[:CPU_SAMPLE_SEQ])
    n = lens[CPU_SAMPLE_SEQ]
    seq = ids[start:start + n].view(1, n)
    mask = torch.ones(1, n)
    times = []
    with torch.no_grad():
        t0 = time.perf_counter()
        model(input_ids=seq, attention_mask=mask)
        first = time.perf_counter() - t0
        w_left = max(0, warmup - 1)
        if first * (w_left + steps) > budget_s:  # keep the whole arm within its time budget
            w_left = min(w_left, 1)
            steps = max(1, min(steps, int((budget_s - first * (1 + w_left)) / max(first, 1e-3))))
        for _ in range(w_left):
            model(input_ids=seq, attention_mask=mask)
        for _ in range(steps):
            t0 = time.perf_counter()
            model(input_ids=seq, attention_mask=mask)
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    return n / (ms / 1e3), ms, len(times), threads, n


def cpu_attention_layer_c1():
    """The CPU-runnable configuration in full: one DeBERTa-v3-base disentangled self-attention layer (transformers' eager
    module, the class the reference falls back to), fp32, batch 2 x 512, seed 0; 3 warm-up + 10 timed calls."""
    from transformers.models.deberta_v2.modeling_deberta_v2 import DisentangledSelfAttention
    torch.set_num_threads(max(1, usable_cores()))
    g = torch.Generator(device="cpu").manual_seed(0)
    layer = DisentangledSelfAttention(deberta_config("base", pos_att_type=["c2p", "p2c"], max_relative_positions=512)).eval()
    with torch.no_grad():
        for p in layer.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.02)
    B, L, hid = 2, 512, 768
    x = torch.randn(B, L, hid, generator=g)
    rel = torch.randn(512, hid, generator=g) * 0.02
    mask = torch.ones(B, 1, L, L)
    times = []
    with torch.no_grad():
        for _ in range(3):
            layer(x, mask, rel_embeddings=rel)
        for _ in range(10):
            t0 = time.perf_counter()
            layer(x, mask, rel_embeddings=rel)
            times.append(time.perf_counter() - t0)
    ms = 1e3 * statistics.median(times)
    f_attn = attn_flops([L] * B, 12)
    f_proj = 3 * 2 * B * L * hid * hid + 2 * 2 * 512 * hid * hid
    return {"ms_median": ms, "tokens_per_s": B * L / (ms / 1e3), "attn_gflops": f_attn / (ms / 1e3) / 1e9,
            "with_projections_gflops": (f_attn + f_proj) / (ms / 1e3) / 1e9, "threads": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "protocol": "batch 2 x 512, fp32, 3 warm-up + 10 timed calls, median"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, ms, steps, threads, n = cpu_eager_encoder(args.steps, args.warmup, budget_s=150.0)
    sample = (f"sequence {CPU_SAMPLE_SEQ} of the batch ({n} tokens) through the full 24-layer fp32 eager encoder "
              "(transformers' DebertaV2Model) per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
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
def dist_setup():
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return dist, rank, world, local_rank, dev


def gpu_arm(args):
    from flashdeberta_b200 import ops
    from flashdeberta_b200.dist import ShardPlan, gather_packed, quadratic_weight_from_times
    from flashdeberta_b200.model import FlashDebertaV2Model

    dist, rank, world, local_rank, dev = dist_setup()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce(x: float, op) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return t.item()

    torch.manual_seed(2)  # same weights on every rank
    model = FlashDebertaV2Model(deberta_config("large", attn_backend="b200")).eval().to(dev).to(torch.bfloat16)
    lens, ids_all = packed_batch()
    assert sum(lens) == 350907 and lens[:8] == [5491, 102, 1993, 880, 5377, 820, 114, 233]
    total, hid = sum(lens), 1024
    warmup = max(args.warmup, 3)
    copy_stream = torch.cuda.Stream(device=dev)

    class Shard:
        """This rank's share under one plan: its ids on the host (pinned) and on the device, its cu_seqlens."""

        def __init__(self, plan):
            self.plan = plan
            self.ids_host = ids_all[plan.local_rows(rank)].contiguous().pin_memory()
            self.cu_host = torch.tensor(plan.cu_seqlens(rank), dtype=torch.int32).pin_memory()
            self.ids_dev, self.cu_dev = self.ids_host.to(dev), self.cu_host.to(dev)
            self.max_len = plan.max_seqlen(rank)
            self.lens = [lens[i] for i in plan.bins[rank]]

        def forward(self, ids, cu):
            h = model(input_ids=ids.view(1, -1), cu_seqlens=cu, max_seqlen=self.max_len).last_hidden_state[0]
            return gather_packed(h, self.plan)

    out_host = torch.empty(total, hid, dtype=torch.bfloat16).pin_memory() if rank == 0 else None

    def step_resident(sh):
        return sh.forward(sh.ids_dev, sh.cu_dev)

    def step_e2e(sh):
        # ids and cu_seqlens come from pinned host memory; the gathered result goes back to pinned host memory on rank 0,
        # on a second stream, so the copy of one step runs beside the next step's kernels (the last copy is waited for
        # before the clock stops, see `timed`)
        out = sh.forward(sh.ids_host.to(dev, non_blocking=True), sh.cu_host.to(dev, non_blocking=True))
        if rank == 0:
            done = torch.cuda.Event()
            done.record()
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(done)
                out_host.copy_(out, non_blocking=True)
            out.record_stream(copy_stream)
        return out

    def timed(fn, sh, steps, log_attention=False):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if log_attention:
            ops.event_log = []
        t0.record()
        for _ in range(steps):
            fn(sh)
        torch.cuda.current_stream().wait_stream(copy_stream)  # the last result has reached the host
        t1.record()
        barrier()
        ms = t0.elapsed_time(t1)
        attn = None
        if log_attention:
            attn = [a.elapsed_time(b) for a, b in ops.event_log]
            ops.event_log = None
        return allreduce(ms, dist.ReduceOp.MAX) if world > 1 else ms, ms, attn

    with torch.no_grad():
        # ---- warm-up 1: token-balanced shards; its timing gives the weight of the quadratic term in a sequence's cost ----
        sh = Shard(ShardPlan(lens, world))
        step_resident(sh)
        _, my_ms, my_attn = timed(step_resident, sh, 1, log_attention=True)
        weight = quadratic_weight_from_times(allreduce(my_ms, dist.ReduceOp.SUM), allreduce(sum(my_attn), dist.ReduceOp.SUM), lens)
        if world > 1:
            sh = Shard(ShardPlan(lens, world, quadratic_weight=weight))
        # ---- warm-up 2: the plan that is timed; the gathered result is checked against sequences run on their own ----
        for _ in range(warmup - 1):
            out = step_resident(sh)
        check = {}
        start = [0]
        for n in lens:
            start.append(start[-1] + n)
        for b in (1, 3, 7):  # three short sequences (102, 880, 233 tokens), whoever owns them
            one = model(input_ids=ids_all[start[b]:start[b + 1]].to(dev).view(1, -1)).last_hidden_state[0]
            d = (one.float() - out[start[b]:start[b + 1]].float()).abs()
            check[f"seq{b}"] = d.max().item()
        # the attention is bit-identical per sequence whatever the batch; the GEMMs see another row count and may round
        # differently: bf16 encoder outputs (|x| ~ 1) within 0.1
        assert max(check.values()) < 0.1, check

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        l0 = ops.launch_count()
        ms_total, _, attn_ms = timed(step_resident, sh, args.steps, log_attention=True)
        launches = ops.launch_count() - l0
        for _ in range(2):
            step_e2e(sh)
        ms_e2e, _, _ = timed(step_e2e, sh, args.steps)
        clocks = sampler.stop() if rank == 0 else None
        ops.check_status(dev)

    ms_step = ms_total / args.steps
    value = total / (ms_step / 1e3)
    e2e_value = total / (ms_e2e / args.steps / 1e3)
    launches_all = int(allreduce(float(launches), dist.ReduceOp.SUM)) if world > 1 else launches
    h2d = int(allreduce(float(sh.ids_host.numel() * 8 + sh.cu_host.numel() * 4), dist.ReduceOp.SUM))
    tok_max = max(sh.plan.tokens)
    f_rank = [attn_flops([lens[i] for i in b], 16) for b in sh.plan.bins]

    # roofline of the fused attention: one launch = one layer's attention over rank 0's own sequences
    f_launch = attn_flops(sh.lens, heads=16)
    attn_avg_ms = sum(attn_ms) / len(attn_ms)
    achieved = f_launch / (attn_avg_ms / 1e3) / 1e12
    peaks = measured_peaks()
    at_max = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and
                  clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"] and "sw_power_cap" not in clocks.get("reasons", []))
    peak = peaks["burst"] if at_max else peaks["sustained"]
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "attn_fwd_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f).get("dram_bytes_per_launch")
    total_flops = 24 * attn_flops(lens, 16) + encoder_linear_flops(total, 1024, 4096, 24)

    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "total_tokens": total, "sequences": len(lens), "tokens_rank0": sh.plan.tokens[0],
                   "parallelism": f"dp{world}: whole sequences per rank, cost = tokens + {weight:.3e} * tokens^2 (weight "
                                  "measured in the warm-up), one final all-gather of packed rows",
                   "token_imbalance": tok_max / (total / world), "attention_flop_imbalance": max(f_rank) / (sum(f_rank) / world),
                   "l2": "per-step working set (weights 0.9 GB + activations) exceeds the 126 MB L2; no explicit flush"},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": total * hid * 2,
                "note": "every rank copies its ids and cu_seqlens in; rank 0 copies the gathered (tokens, 1024) bf16 result out"},
        "gpu_launches": launches_all,
        "clocks": clocks,
        "roofline": {"kernel": "attn_fwd_kernel (+ attn_fwd_far1_kernel for sequences of 3584 tokens or more)", "bound": "tensor",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
                     "peak_source": f"{peaks['source']}, {'burst' if at_max else 'sustained'} figure "
                                    f"({'SM clock at its maximum, no power cap' if at_max else 'SM clock below its maximum or power cap active'})",
                     "frac_of_burst": achieved / peaks["burst"], "frac_of_sustained": achieved / peaks["sustained"],
                     "launch_ms": attn_avg_ms, "flops_per_launch": f_launch,
                     "note": "events bracket one fdb_attn_fwd call on rank 0 (one layer over its own packed sequences)"},
        "attention_share_of_step": attn_avg_ms * 24 / ms_step,
        "model_tflops": total_flops / (ms_step / 1e3) / 1e12,
        "gather_check_max_abs_vs_alone": check,
    }
    if rank == 0 and world == 1:
        if not args.no_extras:
            model = None  # make room for the extra measurements
            torch.cuda.empty_cache()
            line["extra"] = extras(args)
        if not args.no_cpu_baseline:
            tps, ms, steps, threads, n = cpu_eager_encoder(2, 1, budget_s=40.0)
            line["cpu_baseline"] = {
                "value": tps, "unit": "tokens/s", "cores": threads, "kind": "reference", "host_cpus": os.cpu_count(),
                "sample": f"sequence {CPU_SAMPLE_SEQ} of the batch ({n} tokens), full 24-layer fp32 eager encoder "
                          f"(transformers' DebertaV2Model), {steps} step(s)"}
            if not args.no_extras:
                line["extra"]["cpu_c1"] = cpu_attention_layer_c1()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def c2_measure(steps: int, warmup: int, dev):
    """DeBERTa-v3-base encoder, batch 8 x 2048, mask all ones, bf16: (tokens/s resident, ms/step, attention ms/launch)."""
    from flashdeberta_b200 import ops
    from flashdeberta_b200.model import FlashDebertaV2Model
    torch.manual_seed(1)
    model = FlashDebertaV2Model(deberta_config("base", attn_backend="b200")).eval().to(dev).to(torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(1)
    ids = torch.randint(1, 128100, (8, 2048), generator=g).to(dev)
    mask = torch.ones(8, 2048, dtype=torch.long, device=dev)
    with torch.no_grad():
        for _ in range(max(warmup, 3)):
            model(input_ids=ids, attention_mask=mask)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ops.event_log = []
        t0.record()
        for _ in range(steps):
            model(input_ids=ids, attention_mask=mask)
        t1.record()
        torch.cuda.synchronize()
        attn = [a.elapsed_time(b) for a, b in ops.event_log]
        ops.event_log = None
    ms = t0.elapsed_time(t1) / steps
    return 8 * 2048 / (ms / 1e3), ms, sum(attn) / len(attn)


def attention_alone(B: int, L: int, H: int, dev, iters: int = 20, sets: int = 4):
    """The fused attention by itself (c2p + p2c, bf16) on rotated inputs: median ms and algorithmic TFLOP/s."""
    from flashdeberta_b200 import ops
    g = torch.Generator(device="cpu").manual_seed(0)
    data = [tuple(torch.randn(B, L, H, 64, generator=g).bfloat16().to(dev) for _ in range(3)) for _ in range(sets)]
    pk, pq = (torch.randn(H, 512, 64, generator=g).mul_(0.5).bfloat16().to(dev) for _ in range(2))
    kw = dict(max_seqlen=L, position_buckets=256, max_relative_positions=512)
    for i in range(5):
        ops.disentangled_attention(*data[i % sets], pk, pq, **kw)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.disentangled_attention(*data[i % sets], pk, pq, **kw)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    med = statistics.median(times)
    return med, attn_flops([L] * B, H) / med / 1e9


def extras(args):
    dev = torch.device("cuda", torch.cuda.current_device())
    tps, ms, attn_ms = c2_measure(args.steps, args.warmup, dev)
    peaks = measured_peaks()
    f2048 = attn_flops([2048] * 8, 12)
    med, tf = attention_alone(4, 4096, 12, dev)
    return {
        "c2_tokens_per_s": tps, "c2_ms_per_step": ms,
        "c2_workload": "DeBERTa-v3-base encoder fwd, random-init, 12 layers, batch 8 x seq 2048, mask all ones, bf16, ids resident",
        "c2_attn_ms_per_launch": attn_ms, "c2_attn_tflops": f2048 / (attn_ms / 1e3) / 1e12,
        "c2_attn_frac_of_burst": f2048 / (attn_ms / 1e3) / 1e12 / peaks["burst"],
        "attn_seq4096_ms": med, "attn_seq4096_tflops": tf, "attn_seq4096_frac_of_burst": tf / peaks["burst"],
        "attn_seq4096_workload": "fused attention alone, 4 x 4096 x 12 heads, c2p + p2c, bf16, four rotated input sets",
    }


def c2_run(args):
    """The DeBERTa-v3-base 8 x 2048 step as its own JSON line (one GPU)."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tps, ms, attn_ms = c2_measure(args.steps, args.warmup, dev)
    print(json.dumps({"metric": "deberta_v3_base_encoder_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": 1,
                      "steps": args.steps, "ms_per_step": ms, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "DeBERTa-v3-base encoder fwd, random-init, 12 layers, batch 8 x seq 2048, mask all ones"},
                      "attn_ms_per_launch": attn_ms,
                      "attn_tflops": attn_flops([2048] * 8, 12) / (attn_ms / 1e3) / 1e12}), flush=True)


def fp8_run(args):
    """Extra measurement (not the headline line): the e4m3 configuration — DeBERTa-v3-large encoder, random-init, attention
    operands quantised to e4m3 with per-(sequence, head) scales (`config.attn_fp8`), linears in bf16; 64 sequences of 4096
    tokens split evenly over the ranks (16 per GPU at 4 GPUs, 8 per GPU at 8), ids uniform from seed 4; at one or two GPUs
    each rank runs 8 sequences (the per-GPU share at 8 GPUs).  Also times the bf16 attention on the same model and inputs.
    Prints one JSON line with "config": {"workload": "fp8 ..."}."""
    from flashdeberta_b200 import ops
    from flashdeberta_b200.model import FlashDebertaV2Model

    dist, rank, world, local_rank, dev = dist_setup()
    B, L = (64 // world if world >= 4 else 8), 4096

    def build(fp8: bool):
        torch.manual_seed(4)
        return FlashDebertaV2Model(deberta_config("large", attn_backend="b200", attn_fp8=fp8)).eval().to(dev).to(torch.bfloat16)

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
            "n_gpus": world, "steps": args.steps, "ms_per_step": ms8, "scaling": "weak" if world < 4 else "strong",
            "dtype": "e4m3 attention, bf16 linears", "data": "synthetic",
            "config": {"workload": f"fp8: DeBERTa-v3-large encoder, {B} x 4096 tokens per GPU, e4m3 attention operands with "
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
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra one-GPU measurements (8 x 2048 step, attention alone)")
    ap.add_argument("--c2", action="store_true", help="print the DeBERTa-v3-base 8 x 2048 line instead")
    ap.add_argument("--fp8", action="store_true", help="measure the e4m3-attention v3-large configuration instead")
    args = ap.parse_args()
    if args.c2:
        c2_run(args)
    elif args.fp8:
        fp8_run(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
