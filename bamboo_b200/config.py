"""The subset of the DeepSpeed JSON configuration that the pipeline step reads.

Keys and the batch-size rule follow ``deepspeed/runtime/config.py`` of the reference
(batch triad ``:862-932``: ``train_batch_size = micro_batch * gradient_accumulation_steps *
data_parallel_size``; ``optimizer{type, params}``; ``steps_per_print``;
``wall_clock_breakdown``; ``pipeline{...}`` ``:436-447``).  ``bf16{enabled}`` is an addition:
DeepSpeed 0.5.2 has no such key and the sm_100a kernels compute in bf16.
"""
import json
from typing import Optional

RC_MAX_CTAS_DEFAULT = -1
ADAM = "adam"
ADAMW = "adamw"


class DeepSpeedConfigError(Exception):
    pass


class PipeConfig:
    def __init__(self, source, dp_world_size=1):
        if source is None:
            source = {}
        if isinstance(source, str):
            with open(source) as f:
                source = json.load(f)
        self._raw = dict(source)
        tb = self._raw.get("train_batch_size")
        mb = self._raw.get("train_micro_batch_size_per_gpu")
        gas = self._raw.get("gradient_accumulation_steps")
        dp = dp_world_size
        # any two of the three determine the third
        if tb is not None and mb is not None and gas is None:
            gas = tb // (mb * dp)
        elif tb is not None and gas is not None and mb is None:
            mb = tb // (gas * dp)
        elif mb is not None and gas is not None and tb is None:
            tb = mb * gas * dp
        elif tb is not None and mb is None and gas is None:
            gas, mb = 1, tb // dp
        elif mb is not None and tb is None and gas is None:
            gas, tb = 1, mb * dp
        if tb is None or mb is None or gas is None:
            raise DeepSpeedConfigError("Either train_batch_size or micro_batch_per_gpu needs to be provided")
        if tb != mb * gas * dp:
            raise DeepSpeedConfigError(
                f"Check batch related parameters. train_batch_size is not equal to micro_batch_per_gpu * "
                f"gradient_acc_step * world_size {tb} != {mb} * {gas} * {dp}")
        if min(tb, mb, gas) <= 0:
            raise DeepSpeedConfigError("batch sizes must be positive")
        self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps = tb, mb, gas
        opt = self._raw.get("optimizer") or {}
        self.optimizer_name = (opt.get("type") or ADAM).lower()
        self.optimizer_params = dict(opt.get("params") or {})
        self.steps_per_print = int(self._raw.get("steps_per_print", 10))
        self.wall_clock_breakdown = bool(self._raw.get("wall_clock_breakdown", False))
        self.bf16_enabled = bool((self._raw.get("bf16") or {}).get("enabled", False))
        self.fp16_enabled = bool((self._raw.get("fp16") or {}).get("enabled", False))
        pipe = dict(self._raw.get("pipeline") or {})
        pipe.setdefault("stages", "auto")
        pipe.setdefault("partition", "best")
        pipe.setdefault("seed_layers", False)
        pipe.setdefault("activation_checkpoint_interval", 0)
        self.pipeline = pipe
        self.zero_stage = int((self._raw.get("zero_optimization") or {}).get("stage", 0))
        self.gradient_clipping = float(self._raw.get("gradient_clipping", 0.0))
        self.prescale_gradients = bool(self._raw.get("prescale_gradients", False))
        # extension keys of this implementation
        ext = dict(self._raw.get("bamboo_b200") or {})
        self.rc_retain_graph = bool(ext.get("rc_retain_graph", True))
        self.p2p_timeout_s = float(ext.get("p2p_timeout_s", 30.0))
        self.rc_stream_priority_low = bool(ext.get("rc_low_priority_stream", True))
        self.main_stream_high_priority = bool(ext.get("main_stream_high_priority", True))
        # redundant-computation GEMMs as one tile per CTA instead of persistent CTAs (so that a main-
        # stream kernel never waits for a whole tile loop).  Off: measured on 2 GPUs it cost 4 %
        # (308 ms vs 296 ms per step) - the shorter wait does not pay for the slower GEMMs.
        self.rc_short_ctas = bool(ext.get("rc_short_ctas", False))
        # SM budget of a redundant-computation GEMM: 0 = every SM (persistent CTAs, like the main
        # stream's), n > 0 = at most n CTAs, -1 = one work unit per CTA.  Default -1: a low-priority
        # CTA is not preempted, so it should be short-lived - the own stage's next kernel then finds
        # its SMs within microseconds (4 stages, 12-step runs: 156.9 ms/step vs 158.6 with persistent CTAs).
        v = int(ext.get("rc_max_ctas", RC_MAX_CTAS_DEFAULT))
        self.rc_max_ctas = RC_MAX_CTAS_DEFAULT if v == -2 else v
        self.shadow_sync = bool(ext.get("shadow_sync", True))
        # redundant forwards are handed to the GPU layer by layer while the host waits for a
        # neighbour's message with the main stream drained, the remainder at the end of the batch
        self.rc_deferred = bool(ext.get("rc_deferred", True))
        self.rc_chunks_in_flight = int(ext.get("rc_chunks_in_flight", 2))

    def adam_args(self):
        p = self.optimizer_params
        betas = p.get("betas", (0.9, 0.999))
        # the reference builds FusedAdam with adam_w_mode=True unless torch_adam/adam_w_mode say otherwise
        # (deepspeed/runtime/engine.py:973-1008, config.py:50-51)
        return dict(lr=float(p.get("lr", 1e-3)), beta1=float(betas[0]), beta2=float(betas[1]),
                    eps=float(p.get("eps", 1e-8)), weight_decay=float(p.get("weight_decay", 0.0)),
                    adam_w_mode=bool(p.get("adam_w_mode", True)) or self.optimizer_name == ADAMW,
                    bias_correction=bool(p.get("bias_correction", True)))
