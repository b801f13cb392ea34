"""Benchmark of the pipeline training step: tokens/s of GPT-2-medium (24 layers, hidden 1024,
16 heads, FFN 4096, seq 1024, vocab 50257, bf16 with fp32 master weights; micro-batch 8 x 16
micro-batches per step) split over N pipeline stages on N GPUs.

    python bench.py --gpus N --steps K --warmup W [--rc off|lazy|eager] [--impl reference]

One rank per GPU (torchrun for N > 1).  Prints one JSON line on rank 0.  ``value`` is the
device-resident throughput (tokens already in HBM), ``e2e`` is measured through the public
API (``train_batch``) with pinned host token buffers copied in and the loss read back every
step.  ``--impl reference`` times the CPU restatement of the reference's step (the oracle)
on the host cores for the same workload, on a bounded sample per step.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tokens/sec"
MICRO_BATCH, MICRO_BATCHES = 8, 16


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bamboo_b200", choices=["bamboo_b200", "reference"])
    ap.add_argument("--rc", default="auto", choices=["auto", "off", "lazy", "eager"])
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "bert-large", "toy"],
                    help="gpt2-medium is the headline configuration (micro-batch 8 x 16, seq 1024); bert-large is the "
                         "masked-LM configuration (micro-batch 16 x 32, seq 512, bidirectional attention)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--failover", action="store_true",
                    help="after the timed region: the last stage announces its preemption and leaves; reports the "
                         "pause of the first step after it and the post-failover throughput")
    ap.add_argument("--whole-blocks", action="store_true",
                    help="multi-stage runs: keep every transformer block one pipeline layer (coarser stage boundaries)")
    ap.add_argument("--micro-batches", type=int, default=0,
                    help="profiling only: fewer micro-batches per step than the benchmark configuration")
    return ap.parse_args()


def model_config(name):
    from bamboo_b200 import models
    return {"gpt2-medium": models.GPT2_MEDIUM, "bert-large": models.BERT_LARGE}.get(name, models.GPT_TOY)


def contiguous_partition(costs, parts):
    """Boundaries of `parts` non-empty contiguous groups of `costs` with the smallest maximum
    group sum and, among those, the smallest sum of squares (dynamic programme over prefixes).
    The package's `partition_balanced` follows the reference's bottleneck search, which may leave
    the last stages empty when one heavy layer (the vocabulary head) ends the list."""
    n = len(costs)
    pre = [0.0]
    for c in costs:
        pre.append(pre[-1] + c)
    INF = (float("inf"), float("inf"))
    best = [[INF] * (n + 1) for _ in range(parts + 1)]
    arg = [[0] * (n + 1) for _ in range(parts + 1)]
    best[0][0] = (0.0, 0.0)
    for k in range(1, parts + 1):
        for j in range(k, n + 1):
            for i in range(k - 1, j):
                if best[k - 1][i] == INF:
                    continue
                load = pre[j] - pre[i]
                cand = (max(best[k - 1][i][0], load), best[k - 1][i][1] + load * load)
                if cand < best[k][j]:
                    best[k][j], arg[k][j] = cand, i
    bounds, j = [n], n
    for k in range(parts, 0, -1):
        j = arg[k][j]
        bounds.append(j)
    return bounds[::-1]


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synthetic_tokens(cfg, steps, seed, pin):
    """Uniform token ids; labels = tokens shifted by one (last position ignored), or for the
    masked-LM model the BERT masking recipe (15 % of the positions, 80/10/10)."""
    import torch
    from bamboo_b200 import models
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(steps):
        step = []
        for _ in range(MICRO_BATCHES):
            tok = torch.randint(0, cfg.vocab, (MICRO_BATCH, cfg.seq), generator=g)
            if cfg.mlm:
                tok, lab = models.mlm_mask(tok, g, cfg.vocab)
            else:
                lab = torch.full_like(tok, -100)
                lab[:, :-1] = tok[:, 1:]
            if pin:
                tok, lab = tok.pin_memory(), lab.pin_memory()
            step.append((tok, lab))
        out.append(step)
    return out


def cpu_baseline(cfg, seconds_budget=25.0):
    """The oracle (CPU port of the reference step) on the host cores, bounded sample."""
    import torch
    from oracle import gpt_ref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    rc = gpt_ref.RefConfig(cfg.layers, cfg.hidden, cfg.heads, cfg.ffn, cfg.seq, cfg.vocab, cfg.causal, cfg.mlm)
    ref = gpt_ref.RefTrainer(rc, seed=0, lr=1e-4, micro_batches=1)
    g = torch.Generator().manual_seed(1)
    seqs, t_fb = 0, 0.0
    while t_fb < seconds_budget * 0.6 and seqs < 4:
        tok = torch.randint(0, cfg.vocab, (1, cfg.seq), generator=g)
        if cfg.mlm:
            from bamboo_b200 import models
            tok, lab = models.mlm_mask(tok, g, cfg.vocab)
        else:
            lab = torch.full_like(tok, -100); lab[:, :-1] = tok[:, 1:]
        t0 = time.perf_counter()
        loss = gpt_ref.forward_loss(rc, ref.P, tok, lab)
        loss.backward()
        t_fb += time.perf_counter() - t0
        seqs += 1
    t0 = time.perf_counter()
    with torch.no_grad():
        for k, p in ref.P.items():
            gpt_ref.adam_update(p, p.grad, ref.m[k], ref.v[k], 1, 1e-4)
    t_adam = time.perf_counter() - t0
    step_seqs = MICRO_BATCH * MICRO_BATCHES
    per_seq = t_fb / seqs + t_adam / step_seqs
    return {"value": cfg.seq / per_seq, "unit": METRIC, "cores": cores, "kind": "port",
            "sample": f"{seqs} sequence(s) of {cfg.seq} tokens forward+backward in fp32 plus one Adam update "
                      f"amortised over the {step_seqs}-sequence step"}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = model_config(args.model)
    vals = []
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        b = cpu_baseline(cfg, seconds_budget=8.0)
        if i >= args.warmup:
            vals.append(b["value"])
        if time.perf_counter() - t_all > 240:
            break
    v = sum(vals) / max(len(vals), 1) if vals else b["value"]
    b["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": METRIC, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": cfg.seq * MICRO_BATCH * MICRO_BATCHES / v * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.model} pipeline step, micro-batch {MICRO_BATCH} x {MICRO_BATCHES}, seq {cfg.seq}"},
            "cpu_baseline": b, "e2e": {"value": v, "unit": METRIC, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    global MICRO_BATCH, MICRO_BATCHES
    args = parse()
    if args.model == "bert-large":
        MICRO_BATCH, MICRO_BATCHES = 16, 32
    if args.micro_batches:
        MICRO_BATCHES = args.micro_batches
    if args.impl == "reference":
        return run_reference(args)
    import torch
    import torch.distributed as dist
    from bamboo_b200 import api, lib, models
    from bamboo_b200.module import PipelineModule

    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    assert world == args.gpus, f"launch with torchrun --nproc-per-node {args.gpus} (WORLD_SIZE={world})"
    os.environ.setdefault("BAMBOO_QUIET", "1")
    torch.cuda.set_device(local_rank)
    if world > 1:
        api.init_distributed("nccl", rank=rank, world_size=world)
    lib.load()

    cfg = model_config(args.model)
    rc = args.rc if args.rc != "auto" else ("eager" if world > 1 else "off")
    if world == 1:
        rc = "off"
    # stage boundaries balanced by time per micro-batch: a block counts 1, the embedding 0, the
    # vocabulary head its FLOP ratio 2hV / (24h^2 + 4sh) scaled by 0.65, because its three large
    # GEMMs run at ~1.2 PFLOP/s while a block (attention and row-wise kernels included) averages
    # ~0.75 (measured on one GPU: 1.07 ms per block, 2.5 ms for the head, per micro-batch)
    h = cfg.hidden
    blk = 24.0 * h * h + 4.0 * cfg.seq * h
    head_cost = 0.65 * 2.0 * h * cfg.vocab / blk
    # multi-stage runs list every block as two layers (attention half 0.53, MLP half 0.47 of a
    # block's time), so that stage boundaries can fall inside a block: with 24 blocks and a head
    # worth 2.3 blocks, whole blocks leave 8 stages 22 % above the mean load
    split = world > 1 and not args.whole_blocks
    blocks = [0.53, 0.47] * cfg.layers if split else [1.0] * cfg.layers
    costs = [0.0] + blocks + [0.0] + ([0.65 * 2.0 * h * h / blk] if cfg.mlm else []) + [head_cost]
    parts = contiguous_partition(costs, world)
    model = PipelineModule(models.transformer_layer_specs(cfg, 0, split_blocks=split), num_stages=world, loss_fn=models.transformer_loss(cfg),
                           partition_method="custom", custom_partitions=parts)
    engine, *_ = api.initialize(model=model, config={
        "train_micro_batch_size_per_gpu": MICRO_BATCH, "gradient_accumulation_steps": MICRO_BATCHES,
        "bf16": {"enabled": True}, "optimizer": {"type": "Adam", "params": {"lr": 1e-4}},
        "bamboo_b200": {"rc_retain_graph": False, "rc_short_ctas": os.environ.get("BB_RC_SHORT_CTAS", "0") == "1"}},
        redundancy_level=0 if rc == "off" else 1, eager_recovery=(rc == "eager"))
    dev = torch.device("cuda", local_rank)
    tokens_per_step = MICRO_BATCH * MICRO_BATCHES * cfg.seq

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_issue_ms = [0.0]

    def timed(steps_data, read_loss):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        last = None
        t_host = time.perf_counter()
        for batches in steps_data:
            loss = engine.train_batch(data_iter=iter(batches))
            if read_loss and torch.is_tensor(loss):
                last = loss.item()          # device -> host read of the step result
            elif torch.is_tensor(loss):
                last = loss
        end.record()
        # host time to issue the steps, no final sync (an upper bound on the launch cost: a host
        # that runs far ahead blocks on the driver's bounded launch queue and then tracks the GPU)
        host_issue_ms[0] = (time.perf_counter() - t_host) * 1e3
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), last

    host = synthetic_tokens(cfg, max(args.warmup, 1) + args.steps, seed=1, pin=True)
    resident = [[(t.to(dev), l.to(dev)) for t, l in step] for step in host[-args.steps:]]
    timed(host[:max(args.warmup, 1)], read_loss=True)                      # warm-up (untimed)
    if world > 1:
        # multi-stage runs: the caching allocator keeps growing its pools for a few more steps
        # (buffers that crossed to the redundant-computation or weight-gradient stream return
        # late), and every growth is a device-wide cudaMalloc; settle it before the timed region
        timed(host[:max(args.warmup, 1)], read_loss=True)

    sampler = ClockSampler(local_rank)
    sampler.start()
    n0 = lib.LAUNCHES
    ms_dev, loss_dev = timed(resident, read_loss=False)
    issue_ms = host_issue_ms[0] / args.steps
    launches = lib.LAUNCHES - n0
    ms_e2e, loss_e2e = timed(host[-args.steps:], read_loss=True)
    clocks = sampler.stop()
    status = lib.read_status()

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): one extra, instrumented step
    records = []

    def hook(key, flops, launch):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); launch(); e.record()
        records.append((key, flops, s, e))

    from bamboo_b200 import layers as _layers
    lib.gemm_hook = hook
    _layers.WGRAD_SIDE_STREAM = False      # one stream: an event pair brackets exactly one GEMM
    engine.train_batch(data_iter=iter(resident[0]))
    _layers.WGRAD_SIDE_STREAM = True
    lib.gemm_hook = None
    torch.cuda.synchronize()
    g_flops = sum(r[1] for r in records)
    g_ms = sum(r[2].elapsed_time(r[3]) for r in records)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["bf16_tflops_sustained"], "measured (sustained, MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 1400.0, "fallback (sustained)"
    achieved = g_flops / (g_ms * 1e-3) / 1e12 if g_ms > 0 else 0.0
    by_shape = {}
    for key, fl, s, e in records:
        d = by_shape.setdefault(key, [0, 0.0, 0.0]); d[0] += 1; d[1] += fl; d[2] += s.elapsed_time(e)

    failover = None
    if args.failover and world > 1 and rc != "off":
        failover = measure_failover(engine, host, rank, world, tokens_per_step, ms_dev / args.steps)
    if rank != 0:
        if failover is not None:
            sys.stdout.flush()
            os._exit(0)        # the job lost a rank: skip collective teardown
        return
    h2d = sum(t.numel() * t.element_size() + l.numel() * l.element_size() for t, l in host[-1])
    value = tokens_per_step * args.steps / (ms_dev * 1e-3)
    e2e = tokens_per_step * args.steps / (ms_e2e * 1e-3)
    step_flops = cfg.flops_per_token() * tokens_per_step
    line = {
        "metric": METRIC, "value": value, "unit": METRIC, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.model} ({cfg.layers} layers, hidden {cfg.hidden}, seq {cfg.seq}, vocab {cfg.vocab}) "
                               f"pipeline step, {world} stage(s) x 1 replica, micro-batch {MICRO_BATCH} x {MICRO_BATCHES}",
                   "rc": rc, "parallelism": f"pp{world}", "stage_boundaries": parts, "global_batch": MICRO_BATCH * MICRO_BATCHES, "seq_len": cfg.seq,
                   "l2": "working set per step is far larger than L2 (no flush needed)"},
        "e2e": {"value": e2e, "unit": METRIC, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches, "host_issue_ms_per_step": issue_ms, "clocks": clocks, "device_status": status,
        "loss": float(loss_e2e) if loss_e2e is not None else None,
        "model_tflops_per_gpu": step_flops * args.steps / (ms_dev * 1e-3) / 1e12 / world,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": None, "kernel": "gemm_bf16_tcgen05_kernel", "peak_source": peak_src,
                     "launches_per_step": len(records), "gemm_ms_per_step": g_ms,
                     "note": "sum of algorithmic 2MNK over every GEMM launch of one step / sum of their CUDA-event durations "
                             "(instrumented step, weight-gradient side stream folded into the main stream)"},
    }
    if failover is not None:
        line["failover"] = failover
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line), flush=True)
    for key, (n, fl, ms) in sorted(by_shape.items(), key=lambda kv: -kv[1][2]):
        print(f"# gemm M{key[0]} N{key[1]} K{key[2]} a_mn{key[3]} b_mn{key[4]} epi{key[5]}: {n} launches, {ms:.2f} ms, "
              f"{fl / ms / 1e9:.0f} TFLOP/s", file=sys.stderr)


    if failover is not None:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def measure_failover(engine, host, rank, world, tokens_per_step, normal_ms):
    """Host-side fault injection: the rank of the last stage announces its preemption (what its
    SIGTERM handler would do) and exits at the next batch boundary; its predecessor promotes the
    shadow stage.  No collective runs after the announcement.  Times are this rank's own."""
    import torch
    victim = world - 1
    if rank == victim:
        engine.announce_preemption()
    engine.train_batch(data_iter=iter(host[0]))          # last step with the full pipeline
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    try:
        engine.train_batch(data_iter=iter(host[1 % len(host)]))   # victim leaves here; survivors fail over
    except SystemExit:
        # the engine leaves with code 13 (what Bamboo's agent expects); under a plain launcher a
        # non-zero exit would tear the surviving ranks down, so the benchmark reports success
        sys.stdout.flush()
        os._exit(0)
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    post = []
    for i in range(3):
        t0 = time.perf_counter()
        engine.train_batch(data_iter=iter(host[(2 + i) % len(host)]))
        torch.cuda.synchronize()
        post.append(time.perf_counter() - t0)
    post_s = sorted(post)[len(post) // 2]
    return {"victim_stage": victim, "first_step_after_s": first, "normal_step_s": normal_ms * 1e-3,
            "pause_s": max(first - post_s, 0.0), "post_failover_step_s": post_s,
            "post_failover_tokens_per_s": tokens_per_step / post_s,
            "promote_s": engine.timers.get("promote_s", 0.0),
            "definition": "pause = first step after the victim left minus a steady post-failover step"}


if __name__ == "__main__":
    main()
