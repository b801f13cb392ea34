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
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "bert-large", "gpt-6.7b", "resnet152", "toy"],
                    help="gpt2-medium is the headline configuration (micro-batch 8 x 16, seq 1024); bert-large is the "
                         "masked-LM configuration (micro-batch 16 x 32, seq 512, bidirectional attention)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-failover", action="store_true",
                    help="multi-stage runs with redundancy end with a failover measurement (after the timed region one "
                         "stage announces its preemption and leaves; the pause of the first step after it and the "
                         "post-failover throughput are reported); this flag skips it")
    ap.add_argument("--failover", action="store_true", help="accepted for compatibility: the measurement is on by default")
    ap.add_argument("--no-rc-off-arm", action="store_true",
                    help="skip the RC-off pass that multi-stage runs do first to report the RC overhead")
    ap.add_argument("--rc-retain-graph", action="store_true",
                    help="redundant forwards keep their autograd graph, as the reference's shadow forwards do")
    ap.add_argument("--rc-max-ctas", type=int, default=-2,
                    help="SM budget of a redundant-computation GEMM (see bamboo_b200.rc_max_ctas; -2 = library default)")
    ap.add_argument("--rc-frac", type=float, default=0.12,
                    help="eager RC: weight of the next stage's cost in a rank's load when the stage boundaries are "
                         "chosen (1/3 = the redundant forward at full price, 0 = ignore it; most of it hides in idle time)")
    ap.add_argument("--rc-blind-partition", action="store_true",
                    help="eager RC: balance the stages alone (default: balance own stage + redundant forward of the next)")
    ap.add_argument("--engine-options", default="{}",
                    help="JSON object merged into the engine's bamboo_b200 configuration section (A/B measurements)")
    ap.add_argument("--dp", type=int, default=0, help="pipeline replicas (default 1; 2 for gpt-6.7b on 8 GPUs)")
    ap.add_argument("--whole-blocks", action="store_true",
                    help="multi-stage runs: keep every transformer block one pipeline layer (coarser stage boundaries)")
    ap.add_argument("--micro-batches", type=int, default=0,
                    help="profiling only: fewer micro-batches per step than the benchmark configuration")
    return ap.parse_args()


class ResNetBench:
    """ResNet-152 workload (BASELINE configuration 4): 224 x 224 images, 1000 classes, micro-batch
    32 x 16; the unit of throughput is a sample."""
    blocks, classes, size, width = (3, 8, 36, 3), 1000, 224, 64
    seq, mlm, layers, hidden, vocab = 1, False, 50, 2048, 1000          # fields the shared code reads

    def flops_per_token(self):
        from bamboo_b200 import resnet
        return 3 * resnet.conv_flops_per_image(self.blocks, self.size, self.classes, self.width)

    def layer_costs(self):
        """Relative cost of every pipeline layer (stem, 50 blocks, head): its convolution FLOPs."""
        from bamboo_b200 import resnet
        def upto(nblocks):            # FLOPs of the network truncated after `nblocks` bottlenecks (no head)
            done, out = 0, []
            for n in self.blocks:
                take = min(n, nblocks - done)
                if take <= 0:
                    break
                out.append(take); done += take
            return resnet.conv_flops_per_image(tuple(out), self.size, 8, self.width) if out else None
        stem = resnet.conv_flops_per_image((), self.size, 8, self.width)
        costs, prev = [stem], stem
        for i in range(1, sum(self.blocks) + 1):
            cur = upto(i)
            # the truncated count adds a tiny 8-class head on top of the last block's channels: negligible
            costs.append(max(cur - prev, 0)); prev = cur
        costs.append(2 * 2048 * self.classes)
        unit = sum(costs) / len(costs)
        return [c / unit for c in costs]


def model_config(name):
    from bamboo_b200 import models
    if name == "resnet152":
        return ResNetBench()
    return {"gpt2-medium": models.GPT2_MEDIUM, "bert-large": models.BERT_LARGE, "gpt-6.7b": models.GPT_6_7B}.get(name, models.GPT_TOY)


def contiguous_partition(costs, parts, rc_frac=0.0):
    """Boundaries of `parts` non-empty contiguous groups of `costs` with the smallest maximum
    stage load and, among those, the smallest sum of squared loads.  The load of a stage is its
    own cost plus `rc_frac` x the cost of the stage after it: with eager redundant computation a
    rank also runs its successor's forward (a third of that stage's forward+backward time),
    except the last rank, whose shadow stage is never run ahead.  `rc_frac` = 0 balances the
    stages themselves.  (The package's `partition_balanced` follows the reference's bottleneck
    search, which may leave the last stages empty when one heavy layer - the vocabulary head -
    ends the list.)  Dynamic programme over (groups so far, start and end of the last group)."""
    n = len(costs)
    pre = [0.0]
    for c in costs:
        pre.append(pre[-1] + c)
    INF = (float("inf"), float("inf"))
    # best[k][i][j]: k groups cover costs[:j], the last one is costs[i:j]; its own load is still
    # open (it depends on the group after it), the value covers the k-1 groups before it
    best = [dict() for _ in range(parts + 1)]
    for j in range(1, n - parts + 2):
        best[1][(0, j)] = ((0.0, 0.0), None)
    for k in range(2, parts + 1):
        for (h, i), (val, _) in best[k - 1].items():
            for j in range(i + 1, n - (parts - k) + 1):
                prev_load = (pre[i] - pre[h]) + rc_frac * (pre[j] - pre[i])
                cand = (max(val[0], prev_load), val[1] + prev_load * prev_load)
                cur = best[k].get((i, j))
                if cur is None or cand < cur[0]:
                    best[k][(i, j)] = (cand, h)
    final, arg = INF, None
    for (i, j), (val, h) in best[parts].items():
        if j != n:
            continue
        load = pre[j] - pre[i]
        cand = (max(val[0], load), val[1] + load * load)
        if cand < final:
            final, arg = cand, (i, j)
    bounds = [n]
    i, j = arg
    for k in range(parts, 0, -1):
        bounds.append(i)
        if k > 1:
            h = best[k][(i, j)][1]
            i, j = h, i
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


def synthetic_tokens(cfg, steps, seed, pin, replicas=1):
    """Uniform token ids; labels = tokens shifted by one (last position ignored), or for the
    masked-LM model the BERT masking recipe (15 % of the positions, 80/10/10).  Returns
    ``[step][replica][micro_batch] -> (tokens, labels)``."""
    import torch
    from bamboo_b200 import models
    g = torch.Generator().manual_seed(seed)
    out = []
    if isinstance(cfg, ResNetBench):
        # N(0, 1) images in the kernels' input layout ([N, H, W, 8] bf16: 3 image channels, 5 zero
        # planes), uniform labels.  One set of micro-batches serves every step (400 MB of pinned
        # memory per step otherwise); the data never repeats inside a step.
        step = []
        for _ in range(MICRO_BATCHES * replicas):
            img = torch.zeros(MICRO_BATCH, cfg.size, cfg.size, 8, dtype=torch.bfloat16)
            img[..., :3] = torch.randn(MICRO_BATCH, cfg.size, cfg.size, 3, generator=g).to(torch.bfloat16)
            lab = torch.randint(0, cfg.classes, (MICRO_BATCH,), generator=g)
            if pin:
                img, lab = img.pin_memory(), lab.pin_memory()
            step.append((img, lab))
        per_replica = [step[r * MICRO_BATCHES:(r + 1) * MICRO_BATCHES] for r in range(replicas)]
        return [per_replica for _ in range(steps)]
    for _ in range(steps):
        per_replica = []
        for _ in range(replicas):
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
            per_replica.append(step)
        out.append(per_replica)
    return out


def cpu_baseline(cfg, seconds_budget=25.0):
    """The oracle (CPU port of the reference step) on the host cores, bounded sample: a few
    sequences forward+backward in fp32 and one Adam update over all parameters.  ``value`` is the
    whole-step rate those figures imply (extrapolated: the sample is not a whole step)."""
    import torch
    from oracle import gpt_ref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    if isinstance(cfg, ResNetBench):
        from oracle import resnet_ref
        ref = resnet_ref.RefTrainer(cfg.blocks, cfg.classes, cfg.width, seed=0, lr=1e-4, micro_batches=1)
        t_wall = time.perf_counter()
        n = 4
        batch = resnet_ref.synthetic_batches(n, 1, 1, size=cfg.size, classes=cfg.classes, seed=1)[0]
        t0 = time.perf_counter()
        ref.train_batch(batch)
        dt = time.perf_counter() - t0
        return {"value": n / dt, "unit": METRIC, "cores": cores, "kind": "port", "extrapolated": True,
                "sample_ms": (time.perf_counter() - t_wall) * 1e3, "sample_tokens": n,
                "sample": f"one fp32 step over {n} images of {cfg.size} x {cfg.size} (forward, backward, Adam update); "
                          "batch statistics over 4 images instead of 32"}
    rc = gpt_ref.RefConfig(cfg.layers, cfg.hidden, cfg.heads, cfg.ffn, cfg.seq, cfg.vocab, cfg.causal, cfg.mlm)
    ref = gpt_ref.RefTrainer(rc, seed=0, lr=1e-4, micro_batches=1)
    g = torch.Generator().manual_seed(1)
    seqs, t_fb = 0, 0.0
    t_wall = time.perf_counter()
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
    sample_ms = (time.perf_counter() - t_wall) * 1e3
    step_seqs = MICRO_BATCH * MICRO_BATCHES
    per_seq = t_fb / seqs + t_adam / step_seqs
    return {"value": cfg.seq / per_seq, "unit": METRIC, "cores": cores, "kind": "port", "extrapolated": True,
            "sample_ms": sample_ms, "sample_tokens": seqs * cfg.seq,
            "sample": f"{seqs} sequence(s) of {cfg.seq} tokens forward+backward in fp32 plus one Adam update over all "
                      f"parameters; value = seq / (fwd+bwd time per sequence + Adam time / {step_seqs} sequences per step)"}


def cpu_baseline_c1():
    """The CPU-runnable configuration in full: the oracle trains the 4-layer decoder (hidden 256,
    seq 128, vocab 1024, micro-batch 4 x 4, fp32) for its 5 steps in one process."""
    import torch
    from oracle import gpt_ref
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    cfg = gpt_ref.RefConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=1e-4, micro_batches=4)
    data = gpt_ref.synthetic_batches(cfg, 4, 4, 5, seed=1)
    t0 = time.perf_counter()
    losses = [ref.train_batch(b) for b in data]
    dt = time.perf_counter() - t0
    return {"value": 5 * 4 * 4 * 128 / dt, "unit": METRIC, "cores": cores, "kind": "port", "extrapolated": False,
            "steps": 5, "seconds": dt, "first_loss": losses[0], "last_loss": losses[-1],
            "sample": "5 full steps of the 2-stage plumbing configuration's model (2048 tokens each), single process"}


def run_reference(args):
    """Reference arm: the oracle port on the host cores.  A 'step' here is one bounded sample
    (see cpu_baseline); ``ms_per_step`` is the wall time of that sample as it ran and ``value``
    the whole-step rate it implies."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = model_config(args.model)
    vals, sample_ms = [], []
    t_all = time.perf_counter()
    for i in range(args.warmup + args.steps):
        b = cpu_baseline(cfg, seconds_budget=8.0)
        if i >= args.warmup:
            vals.append(b["value"]); sample_ms.append(b["sample_ms"])
        if time.perf_counter() - t_all > 200:
            break
    v = sum(vals) / max(len(vals), 1) if vals else b["value"]
    b["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": METRIC, "n_gpus": args.gpus, "steps": len(vals) or 1,
            "warmup": args.warmup, "ms_per_step": (sum(sample_ms) / len(sample_ms)) if sample_ms else b["sample_ms"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.model} pipeline step, micro-batch {MICRO_BATCH} x {MICRO_BATCHES}, seq {cfg.seq}",
                       "step": "one bounded sample of the workload (not a whole step): see cpu_baseline.sample; "
                               "value is extrapolated to the whole-step rate"},
            "cpu_baseline": b, "cpu_baseline_c1": cpu_baseline_c1(),
            "e2e": {"value": v, "unit": METRIC, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def stage_costs(cfg, split):
    """Relative time per micro-batch of every pipeline layer: a block counts 1, the embedding 0, the
    vocabulary head its FLOP ratio 2hV / (24h^2 + 4sh) scaled by 0.65, because its three large
    GEMMs run at ~1.2 PFLOP/s while a block (attention and row-wise kernels included) averages
    ~0.75 (measured on one GPU: 1.07 ms per block, 2.5 ms for the head, per micro-batch).  With
    `split` every block is two layers (attention half 0.53, MLP half 0.47 of a block's time), so
    that stage boundaries can fall inside a block: with 24 blocks and a head worth 2.3 blocks,
    whole blocks leave 8 stages 22 % above the mean load."""
    if isinstance(cfg, ResNetBench):
        return cfg.layer_costs()
    h = cfg.hidden
    blk = 24.0 * h * h + 4.0 * cfg.seq * h
    head_cost = 0.65 * 2.0 * h * cfg.vocab / blk
    blocks = [0.53, 0.47] * cfg.layers if split else [1.0] * cfg.layers
    return [0.0] + blocks + [0.0] + ([0.65 * 2.0 * h * h / blk] if cfg.mlm else []) + [head_cost]


def main():
    global MICRO_BATCH, MICRO_BATCHES
    args = parse()
    if args.model == "bert-large":
        MICRO_BATCH, MICRO_BATCHES = 16, 32
    elif args.model == "gpt-6.7b":
        MICRO_BATCH, MICRO_BATCHES = 2, 32
    elif args.model == "resnet152":
        global METRIC
        METRIC = "samples/sec"
        MICRO_BATCH, MICRO_BATCHES = 32, 16
    if args.micro_batches:
        MICRO_BATCHES = args.micro_batches
    if args.impl == "reference":
        return run_reference(args)
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    assert world == args.gpus, f"launch with torchrun --nproc-per-node {args.gpus} (WORLD_SIZE={world})"
    if world > 1:
        # a rank leaves the job in the failover measurement: no NVLink multicast bindings in this run
        os.environ["NCCL_NVLS_ENABLE"] = "0"
    import gc
    import torch
    import torch.distributed as dist
    from bamboo_b200 import api, lib, models
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.topology import PipeDataParallelTopology

    os.environ.setdefault("BAMBOO_QUIET", "1")
    torch.cuda.set_device(local_rank)
    if world > 1:
        api.init_distributed("nccl", rank=rank, world_size=world)
    lib.load()

    cfg = model_config(args.model)
    dp = args.dp if args.dp else (2 if (args.model == "gpt-6.7b" and world >= 8) else 1)
    assert world % dp == 0
    stages = world // dp
    rc = args.rc if args.rc != "auto" else ("eager" if stages > 1 else "off")
    if stages == 1:
        rc = "off"
    split = stages > 1 and not args.whole_blocks and not isinstance(cfg, ResNetBench)
    def parts_for(arm_rc):
        # with eager RC every rank but the last also runs its successor's forward: that load is
        # balanced; every other arm (RC off, lazy) balances the stages alone
        frac = args.rc_frac if (arm_rc == "eager" and not args.rc_blind_partition) else 0.0
        return contiguous_partition(stage_costs(cfg, split), stages, rc_frac=frac)

    parts = parts_for(rc)
    dev = torch.device("cuda", local_rank)
    tokens_per_step = MICRO_BATCH * MICRO_BATCHES * dp * cfg.seq
    base_store = None
    if world > 1:
        from torch.distributed.distributed_c10d import _get_default_store
        base_store = _get_default_store()

    def build(arm_rc, tag):
        topo = PipeDataParallelTopology(num_pp=stages, num_dp=dp)
        if isinstance(cfg, ResNetBench):
            from bamboo_b200 import resnet
            specs, loss_fn = resnet.resnet_layer_specs(cfg.blocks, cfg.classes, cfg.width, seed=0), resnet.resnet_loss(cfg.classes)
        else:
            specs, loss_fn = models.transformer_layer_specs(cfg, 0, split_blocks=split), models.transformer_loss(cfg)
        model = PipelineModule(specs, topology=topo, loss_fn=loss_fn, partition_method="custom",
                               custom_partitions=parts_for(arm_rc))
        store = dist.PrefixStore(f"bench-{tag}", base_store) if base_store is not None else None
        engine, *_ = api.initialize(model=model, config={
            "train_micro_batch_size_per_gpu": MICRO_BATCH, "gradient_accumulation_steps": MICRO_BATCHES,
            "train_batch_size": MICRO_BATCH * MICRO_BATCHES * dp,
            "bf16": {"enabled": True}, "optimizer": {"type": "Adam", "params": {"lr": 1e-4}},
            "bamboo_b200": dict({"rc_retain_graph": bool(args.rc_retain_graph), "rc_max_ctas": args.rc_max_ctas},
                                **json.loads(args.engine_options))},
            redundancy_level=0 if arm_rc == "off" else 1, eager_recovery=(arm_rc == "eager"), store=store)
        return engine

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_warm = max(args.warmup, 1)
    host_all = synthetic_tokens(cfg, n_warm + args.steps, seed=1, pin=True, replicas=dp)

    def run_arm(arm_rc, tag):
        """Warm-up (twice: the caching allocator keeps growing its pools for a few steps when
        buffers cross to the redundant-computation or weight-gradient stream, and every growth
        is a device-wide cudaMalloc), then K resident steps and K end-to-end steps, timed."""
        engine = build(arm_rc, tag)
        replica = engine.grid.get_data_parallel_id()
        host = [step[replica] for step in host_all]
        resident = [[(t.to(dev), l.to(dev)) for t, l in step] for step in host[-args.steps:]]
        losses = []
        info = {}

        def timed(steps_data, read_loss):
            barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            t_host = time.perf_counter()
            for batches in steps_data:
                loss = engine.train_batch(data_iter=iter(batches))
                if torch.is_tensor(loss):
                    losses.append(loss.item() if read_loss else loss)      # .item(): device -> host read of the step result
                else:
                    losses.append(None)
            end.record()
            # host time to issue the steps, no final sync (an upper bound on the launch cost: a host
            # that runs far ahead blocks on the driver's bounded launch queue and then tracks the GPU)
            info["issue_ms"] = (time.perf_counter() - t_host) * 1e3
            barrier()
            ms = torch.tensor([start.elapsed_time(end)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return ms.item()

        timed(host[:n_warm], read_loss=True)
        timed(host[:n_warm], read_loss=True)
        n0 = lib.LAUNCHES
        wait0 = getattr(engine.transport, "wait_s", 0.0)
        idle0 = getattr(engine.transport, "idle_s", 0.0)
        if hasattr(engine.transport, "measure_idle"):
            engine.transport.measure_idle = True
        c0 = dict(engine.instr_counts)
        ms_dev = timed(resident, read_loss=False)
        idle_ms = (getattr(engine.transport, "idle_s", 0.0) - idle0) * 1e3 / args.steps
        print(f"# rank {rank} arm {arm_rc}: {ms_dev / args.steps:.1f} ms/step, host issue {info['issue_ms'] / args.steps:.1f} ms, "
              f"waiting for messages {(getattr(engine.transport, 'wait_s', 0.0) - wait0) * 1e3 / args.steps:.1f} ms of which "
              f"with the stream drained {idle_ms:.1f} ms; redundant chunks in idle time "
              f"{engine.instr_counts.get('rc_chunks_in_idle_time', 0) - c0.get('rc_chunks_in_idle_time', 0)}, flushed "
              f"{engine.instr_counts.get('rc_chunks_flushed', 0) - c0.get('rc_chunks_flushed', 0)}", file=sys.stderr, flush=True)
        issue_ms = info["issue_ms"] / args.steps
        recv_wait_ms = (getattr(engine.transport, "wait_s", 0.0) - wait0) * 1e3 / args.steps
        launches = lib.LAUNCHES - n0
        ms_e2e = timed(host[-args.steps:], read_loss=True)
        losses = [float(x) if x is not None else None for x in losses]
        return {"engine": engine, "host": host, "resident": resident, "ms_dev": ms_dev, "ms_e2e": ms_e2e,
                "launches": launches, "issue_ms": issue_ms, "recv_wait_ms": recv_wait_ms, "losses": losses,
                "first_timed_loss": losses[2 * n_warm] if len(losses) > 2 * n_warm else None}

    def share_loss(arm, tag):
        """The rank that owns the last stage of replica 0 publishes its losses; rank 0 prints them."""
        if world == 1:
            return arm["losses"]
        eng = arm["engine"]
        key = f"bench-loss-{tag}"
        if eng.is_last_stage() and eng.grid.get_data_parallel_id() == 0:
            base_store.set(key, json.dumps(arm["losses"]))
        if rank == 0:
            base_store.wait([key])
            return json.loads(base_store.get(key).decode())
        return None

    sampler = ClockSampler(local_rank)
    rc_off = None
    if rc != "off" and not args.no_rc_off_arm:
        # the same pipeline without redundancy, back to back, for the RC overhead
        sampler_off = ClockSampler(local_rank)
        sampler_off.start()
        off = run_arm("off", "off")
        clocks_off = sampler_off.stop()
        off_losses = share_loss(off, "off")
        rc_off = {"tokens_per_s": tokens_per_step * args.steps / (off["ms_dev"] * 1e-3), "ms_per_step": off["ms_dev"] / args.steps,
                  "loss": off_losses[2 * n_warm] if off_losses else None, "clocks": clocks_off,
                  "stage_boundaries": parts_for("off")}
        off["engine"].transport.close()
        del off
        gc.collect()
        torch.cuda.empty_cache()
        barrier()
    sampler.start()
    arm = run_arm(rc, rc)
    clocks = sampler.stop()
    engine, host, resident = arm["engine"], arm["host"], arm["resident"]
    ms_dev, ms_e2e = arm["ms_dev"], arm["ms_e2e"]
    all_losses = share_loss(arm, rc)
    status = lib.read_status()

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): one extra, instrumented step
    records = []

    def hook(key, flops, launch):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); launch(); e.record()
        records.append((key, flops, s, e))

    from bamboo_b200 import layers as _layers
    g_flops = g_ms = 0.0
    by_shape = {}
    if world == 1:
        lib.gemm_hook = hook
        _layers.WGRAD_SIDE_STREAM = False      # one stream: an event pair brackets exactly one GEMM
        engine.train_batch(data_iter=iter(resident[0]))
        _layers.WGRAD_SIDE_STREAM = True
        lib.gemm_hook = None
        torch.cuda.synchronize()
        g_flops = sum(r[1] for r in records)
        g_ms = sum(r[2].elapsed_time(r[3]) for r in records)
        for key, fl, s, e in records:
            d = by_shape.setdefault(key, [0, 0.0, 0.0]); d[0] += 1; d[1] += fl; d[2] += s.elapsed_time(e)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["bf16_tflops_sustained"], "measured (sustained, MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 1400.0, "fallback (sustained)"
    step_flops = cfg.flops_per_token() * tokens_per_step
    model_tflops = step_flops * args.steps / (ms_dev * 1e-3) / 1e12 / world
    if world == 1:
        achieved = g_flops / (g_ms * 1e-3) / 1e12 if g_ms > 0 else 0.0
        roof_note = ("sum of algorithmic 2MNK over every GEMM launch of one step / sum of their CUDA-event durations "
                     "(instrumented step, weight-gradient side stream folded into the main stream)")
    else:
        # several streams and ranks overlap here: per-kernel event pairs would time the overlap, so the
        # multi-GPU line reports the whole step's algorithmic model FLOPs per GPU against the same peak
        achieved = model_tflops
        roof_note = "algorithmic model FLOPs of the whole step (dense attention count, RC excluded) / step time / GPUs"

    failover = None
    if not args.no_failover and stages > 1 and rc != "off":
        victim_stage = 2 if (args.model == "gpt-6.7b" and stages >= 4) else stages - 1
        failover = measure_failover(engine, host, world, tokens_per_step, ms_dev / args.steps, victim_stage, dp)
    if rank != 0:
        if failover is not None:
            sys.stdout.flush()
            os._exit(0)        # the job lost a rank: skip collective teardown
        return
    h2d = sum(t.numel() * t.element_size() + l.numel() * l.element_size() for t, l in host[-1]) * dp
    value = tokens_per_step * args.steps / (ms_dev * 1e-3)
    e2e = tokens_per_step * args.steps / (ms_e2e * 1e-3)
    first_loss = all_losses[2 * n_warm] if all_losses and len(all_losses) > 2 * n_warm else None
    line = {
        "metric": METRIC, "value": value, "unit": METRIC, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": (f"resnet152 (bottleneck blocks {list(cfg.blocks)}, {cfg.size} x {cfg.size} x 3 images, {cfg.classes} classes, "
                                 "bf16 channels-last) " if isinstance(cfg, ResNetBench) else
                                 f"{args.model} ({cfg.layers} layers, hidden {cfg.hidden}, seq {cfg.seq}, vocab {cfg.vocab}) ") +
                               f"pipeline step, {stages} stage(s) x {dp} replica(s), micro-batch {MICRO_BATCH} x {MICRO_BATCHES}",
                   "rc": rc, "rc_retain_graph": bool(args.rc_retain_graph),
                   "parallelism": f"pp{stages}" + (f"dp{dp}" if dp > 1 else ""), "stage_boundaries": parts,
                   "global_batch": MICRO_BATCH * MICRO_BATCHES * dp, "seq_len": cfg.seq,
                   "l2": "working set per step is far larger than L2 (no flush needed)"},
        "e2e": {"value": e2e, "unit": METRIC, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * dp,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": arm["launches"], "host_issue_ms_per_step": arm["issue_ms"],
        "host_recv_wait_ms_per_step": arm["recv_wait_ms"], "clocks": clocks, "device_status": status,
        "loss": first_loss, "loss_step": 2 * n_warm,
        "loss_note": "mean micro-batch loss of the first timed step (after 2 x warm-up optimizer steps), read on the rank "
                     "that owns the last stage of replica 0; same seed and step index at every N",
        "model_tflops_per_gpu": model_tflops,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": GEMM_TRAFFIC_BYTES if world == 1 else None,
                     "traffic_note": GEMM_TRAFFIC_NOTE if world == 1 else None,
                     "kernel": "gemm_bf16_tcgen05_kernel", "peak_source": peak_src,
                     "launches_per_step": len(records), "gemm_ms_per_step": g_ms, "note": roof_note},
    }
    if rc_off is not None:
        eager_tps = value
        line["rc_overhead"] = (rc_off["tokens_per_s"] - eager_tps) / rc_off["tokens_per_s"]
        line["rc_off"] = rc_off
        line["rc_note"] = (f"{rc} RC vs the same pipeline without redundancy, back to back in this run; redundant forwards "
                           + ("keep" if args.rc_retain_graph else "do not keep") + " their autograd graph (rc_retain_graph)")
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


# DRAM traffic of the dominant GEMM launch (M8192 N4096 K1024, bias+GeLU epilogue, two bf16
# outputs), dram__bytes_read.sum + dram__bytes_write.sum from the ncu capture summarised in
# profiles/gemm_bf16_tcgen05_M8192_N4096_K1024.md; algorithmic bytes of that launch: 159 MB
GEMM_TRAFFIC_BYTES = 107.5e6
GEMM_TRAFFIC_NOTE = ("bytes per launch of the M8192 N4096 K1024 bias+GeLU GEMM (ncu, profiles/); below the 159 MB of "
                     "algorithmic bytes because the weight operand and part of the activations stay in the 126 MB L2")


def measure_failover(engine, host, world, tokens_per_step, normal_ms, victim_stage, dp):
    """Host-side fault injection: the rank of `victim_stage` in replica 0 announces its preemption
    (what its SIGTERM handler would do) and exits at the next batch boundary, with none of its
    kernels or collectives in flight; its predecessor promotes the shadow stage.  No collective
    over the whole job runs after the announcement.  Times are this rank's own."""
    import torch
    victim = engine.grid._topo.get_rank(pipe=victim_stage, data=0)
    if engine.global_rank == victim:
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
    return {"victim_stage": victim_stage, "victim_rank": victim, "first_step_after_s": first, "normal_step_s": normal_ms * 1e-3,
            "pause_s": max(first - normal_ms * 1e-3, 0.0), "post_failover_step_s": post_s,
            "post_failover_tokens_per_s": tokens_per_step / post_s,
            "post_failover_fraction": (normal_ms * 1e-3) / post_s,
            "promote_s": engine.timers.get("promote_s", 0.0),
            "definition": "pause = wall time of the first step after the victim left (promotion, schedule rebuild, first "
                          "merged step) minus one normal step before the failure; times are rank 0's own"}


if __name__ == "__main__":
    main()
