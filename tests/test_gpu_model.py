"""Per-step loss and gradient parity of the CUDA training step with the fp32 oracle on the
same seeded weights and tokens (bf16 tolerance 2e-2 relative), through the public API
(PipelineModule / deepspeed.initialize / train_batch)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from oracle import gpt_ref  # noqa: E402

pytestmark = pytest.mark.gpu
TOL = 2e-2


def build_engine(cfg, mb, gas, lr, seed=0, ckpt_interval=0, split_blocks=False):
    from bamboo_b200 import api, models
    from bamboo_b200.module import PipelineModule
    os.environ["BAMBOO_QUIET"] = "1"
    tc = models.TransformerConfig(layers=cfg.layers, hidden=cfg.hidden, heads=cfg.heads, ffn=cfg.ffn, seq=cfg.seq,
                                  vocab=cfg.vocab, causal=cfg.causal, mlm=cfg.mlm)
    model = PipelineModule(models.transformer_layer_specs(tc, seed, split_blocks=split_blocks), num_stages=1, loss_fn=models.transformer_loss(tc),
                           partition_method="uniform", activation_checkpoint_interval=ckpt_interval)
    config = {"train_micro_batch_size_per_gpu": mb, "gradient_accumulation_steps": gas, "bf16": {"enabled": True},
              "optimizer": {"type": "Adam", "params": {"lr": lr}}}
    engine, *_ = api.initialize(model=model, config=config)
    engine.capture_grads = True
    return engine


def oracle_names(cfg):
    names = ["wte", "wpe"]
    for i in range(cfg.layers):
        names += [f"b{i}.{n}" for n in ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b",
                                        "fc1_w", "fc1_b", "fc2_w", "fc2_b")]
    names += ["lnf_w", "lnf_b"]
    if cfg.mlm:
        names += ["mlm_w", "mlm_b", "mlm_ln_w", "mlm_ln_b"]
    return names + ["head_w"]


def compare_grads(engine, ref, cfg):
    arena = engine.arenas[0]
    flat = engine.last_grads[0].cpu()
    worst = 0.0
    for (i, off, n), name in zip(arena.named_slices(), oracle_names(cfg)):
        want = ref.last_grads[name]
        got = flat[off:off + n].view(arena.params[i].shape)[: want.shape[0]]
        rel = ((got - want).norm() / (want.norm() + 1e-12)).item()
        worst = max(worst, rel)
        assert rel <= 5 * TOL, (name, rel)        # per-tensor (small bias vectors are noisier)
    got_all = torch.cat([flat[off:off + n].view(arena.params[i].shape)[: ref.last_grads[nm].shape[0]].reshape(-1)
                         for (i, off, n), nm in zip(arena.named_slices(), oracle_names(cfg))])
    want_all = torch.cat([ref.last_grads[nm].reshape(-1) for nm in oracle_names(cfg)])
    assert ((got_all - want_all).norm() / want_all.norm()).item() <= TOL
    return worst


def test_toy_gpt_five_steps_match_oracle():
    """The 2-stage toy of the plumbing configuration, run here as one stage on one GPU:
    4 layers, hidden 256, 4 heads, FFN 1024, seq 128, vocab 1024, micro-batch 4 x 4."""
    cfg = gpt_ref.RefConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
    mb, gas, steps, lr = 4, 4, 5, 1e-4
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr)
    data = gpt_ref.synthetic_batches(cfg, mb, gas, steps, seed=1)
    for batches in data:
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)
    # weights after 5 Adam steps
    arena = engine.arenas[0]
    for (i, off, n), name in zip(arena.named_slices(), oracle_names(cfg)):
        want = ref.P[name].detach()
        got = arena.master[off:off + n].view(arena.params[i].shape)[: want.shape[0]].cpu()
        assert (got - want).abs().max().item() <= 5 * lr * steps * 0.5 + 1e-6, name
    from bamboo_b200 import lib
    torch.cuda.synchronize()
    assert lib.read_status() == 0


def test_bidirectional_ragged_vocab_matches_oracle():
    """Encoder-style attention and a vocabulary that is not a multiple of the tile width."""
    cfg = gpt_ref.RefConfig(layers=2, hidden=128, heads=2, ffn=512, seq=64, vocab=1000, causal=False)
    mb, gas, lr = 2, 2, 1e-3
    ref = gpt_ref.RefTrainer(cfg, seed=3, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr, seed=3)
    for batches in gpt_ref.synthetic_batches(cfg, mb, gas, 2, seed=5):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)


def test_activation_checkpointing_on_gpu_matches_oracle():
    """Every second layer boundary is a checkpoint: the CUDA layers run their forward twice (the
    cross-entropy gradient, written in place over the logits, then lands in the recomputed copy)."""
    cfg = gpt_ref.RefConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
    mb, gas, lr = 4, 2, 1e-3
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr, ckpt_interval=2)
    for batches in gpt_ref.synthetic_batches(cfg, mb, gas, 2, seed=1):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)


def test_split_blocks_equal_fused_blocks():
    """Blocks as two pipeline layers each (attention half, MLP half): same weights, same
    arithmetic, same parameter order - loss and gradients match the oracle like the fused block."""
    cfg = gpt_ref.RefConfig(layers=3, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
    mb, gas, lr = 4, 2, 1e-3
    ref = gpt_ref.RefTrainer(cfg, seed=4, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr, seed=4, split_blocks=True)
    for batches in gpt_ref.synthetic_batches(cfg, mb, gas, 2, seed=1):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)


def test_masked_lm_encoder_matches_oracle():
    """BERT-style configuration at toy size: bidirectional attention, masked-LM head transform
    (dense + GeLU + LayerNorm, stand-alone GeLU backward), loss on the 15 % chosen positions."""
    cfg = gpt_ref.RefConfig(layers=2, hidden=256, heads=4, ffn=1024, seq=128, vocab=1000, causal=False, mlm=True)
    mb, gas, lr = 4, 2, 1e-3
    ref = gpt_ref.RefTrainer(cfg, seed=2, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr, seed=2)
    for batches in gpt_ref.synthetic_mlm_batches(cfg, mb, gas, 3, seed=7):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)
    from bamboo_b200 import lib
    torch.cuda.synchronize()
    assert lib.read_status() == 0


def test_layers_refuse_cpu_tensors():
    from bamboo_b200 import layers, lib
    blk = layers.TransformerBlock(64, 1, 256)
    with pytest.raises(lib.BambooNativeError):
        blk(torch.zeros(1, 8, 64))


# ---------------------------------------------------------------------------------------------
# the benchmark configurations at their own dimensions (depth cut to two blocks so that the fp32
# oracle finishes in seconds on the host): the kernels take the same paths as in the timed runs -
# hidden 1024 with 16 heads of 64, 1024-token causal tiles (16 key sub-blocks per query tile),
# vocabulary 50257 padded to 50304, CTA-pair GEMMs on the K >= 2048 shapes
def test_gpt2_medium_dimensions_match_oracle():
    cfg = gpt_ref.RefConfig(layers=2, hidden=1024, heads=16, ffn=4096, seq=1024, vocab=50257)
    mb, gas, lr = 2, 2, 1e-4
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr)
    for batches in gpt_ref.synthetic_batches(cfg, mb, gas, 2, seed=1):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)
    from bamboo_b200 import lib
    torch.cuda.synchronize()
    assert lib.read_status() == 0


def test_bert_large_dimensions_match_oracle():
    """Masked-LM encoder at its benchmark dimensions: seq 512, bidirectional attention, vocabulary
    30522 padded to 30592, loss on the 15 % chosen positions."""
    cfg = gpt_ref.RefConfig(layers=2, hidden=1024, heads=16, ffn=4096, seq=512, vocab=30522, causal=False, mlm=True)
    mb, gas, lr = 2, 2, 1e-4
    ref = gpt_ref.RefTrainer(cfg, seed=0, lr=lr, micro_batches=gas)
    engine = build_engine(cfg, mb, gas, lr)
    for batches in gpt_ref.synthetic_mlm_batches(cfg, mb, gas, 2, seed=7):
        want = ref.train_batch(batches)
        got = float(engine.train_batch(data_iter=iter(batches)))
        assert got == pytest.approx(want, rel=TOL)
        compare_grads(engine, ref, cfg)
    from bamboo_b200 import lib
    torch.cuda.synchronize()
    assert lib.read_status() == 0


def test_checkpoint_round_trip_on_cuda_arena(tmp_path):
    """Per-layer checkpoint files written from a CUDA parameter arena and loaded into a fresh
    engine: master weights and Adam moments come back bit-identical, the bf16 working copy is
    re-derived, and the next step's loss is the same number."""
    cfg = gpt_ref.RefConfig(layers=2, hidden=256, heads=4, ffn=1024, seq=128, vocab=1000)
    mb, gas, lr = 2, 2, 1e-3
    data = gpt_ref.synthetic_batches(cfg, mb, gas, 3, seed=1)
    a = build_engine(cfg, mb, gas, lr)
    for batches in data[:2]:
        a.train_batch(data_iter=iter(batches))
    ckpt = str(tmp_path / "ckpt")
    a.save_checkpoint(ckpt, client_state={"k": 1})
    want = float(a.train_batch(data_iter=iter(data[2])))
    files = sorted(os.listdir(os.path.join(ckpt, "global_step2")))
    assert files == [f"layer_{i:02d}-model_states.pt" for i in range(5)] + ["mp_rank_00_model_states.pt"]
    b = build_engine(cfg, mb, gas, lr)
    path, client = b.load_checkpoint(ckpt)
    assert path is not None and client == {"k": 1} and b.global_steps == 2
    got = float(b.train_batch(data_iter=iter(data[2])))
    assert got == want
    for name in ("master", "exp_avg", "exp_avg_sq", "lp"):
        assert torch.equal(getattr(a.arenas[0], name), getattr(b.arenas[0], name)), name
