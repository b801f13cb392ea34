"""Layer lists of the benchmark model families (token-input GPT decoder, BERT-style MLM
encoder) for ``PipelineModule``.

The reference's example models (``DeepSpeedExamples/pipeline_parallelism/gpt2.py:20-154``,
``bert.py:20-150``) have no embedding or vocabulary head and train on random activations;
the benchmark configurations ask for token inputs, learned position embeddings, pre-LN
blocks and a cross-entropy loss, so the layer list is:

    TokenEmbedding, TransformerBlock x L, LayerNorm, Linear(hidden -> vocab, no bias)

and for the masked-LM encoder (``mlm=True``: bidirectional attention, loss on the chosen
positions only) the head is the BERT one:

    ..., LayerNorm, MLMTransform(dense + GeLU + LayerNorm), Linear(hidden -> vocab, no bias)

Initialisation: N(0, 0.02) weights, zero biases, unit LayerNorm gains; layer ``i`` of the
list draws from ``torch.Generator().manual_seed(seed * 1000 + i)`` in parameter-definition
order, so a stage (or a shadow copy of it) built on any rank holds identical values.
"""
from dataclasses import dataclass

import torch

from .layers import (AttentionHalf, CrossEntropyLoss, LayerNorm, Linear, MLMTransform, MLPHalf, TokenEmbedding,
                     TransformerBlock)
from .module import LayerSpec


@dataclass
class TransformerConfig:
    layers: int
    hidden: int
    heads: int
    ffn: int
    seq: int
    vocab: int
    causal: bool = True
    vocab_pad: int = 128
    mlm: bool = False

    @property
    def padded_vocab(self):
        return (self.vocab + self.vocab_pad - 1) // self.vocab_pad * self.vocab_pad

    def flops_per_token(self):
        """Training FLOPs per token, dense attention count: 3 * (L*(24h^2 + 4sh) + 2hV), plus
        2h^2 forward for the masked-LM transform (logits are computed at every position)."""
        h = self.hidden
        head = 2 * h * self.vocab + (2 * h * h if self.mlm else 0)
        return 3 * (self.layers * (24 * h * h + 4 * self.seq * h) + head)


GPT_TOY = TransformerConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
GPT2_MEDIUM = TransformerConfig(layers=24, hidden=1024, heads=16, ffn=4096, seq=1024, vocab=50257)
BERT_LARGE = TransformerConfig(layers=24, hidden=1024, heads=16, ffn=4096, seq=512, vocab=30522, causal=False, mlm=True)
BERT_TOY = TransformerConfig(layers=2, hidden=256, heads=4, ffn=1024, seq=128, vocab=1000, causal=False, mlm=True)
GPT_6_7B = TransformerConfig(layers=32, hidden=4096, heads=32, ffn=16384, seq=2048, vocab=50257)


def transformer_layer_specs(cfg: TransformerConfig, seed: int = 0, split_blocks: bool = False):
    """``split_blocks``: every block becomes two pipeline layers (attention half, MLP half) with
    the same weights and arithmetic, so that stage boundaries can fall inside a block."""
    base = seed * 1000
    specs = [LayerSpec(TokenEmbedding, cfg.vocab, cfg.hidden, cfg.seq, seed=base)]
    for i in range(cfg.layers):
        if split_blocks:
            specs.append(LayerSpec(AttentionHalf, cfg.hidden, cfg.heads, cfg.ffn, causal=cfg.causal, seed=base + 1 + i))
            specs.append(LayerSpec(MLPHalf, cfg.hidden, cfg.heads, cfg.ffn, causal=cfg.causal, seed=base + 1 + i))
        else:
            specs.append(LayerSpec(TransformerBlock, cfg.hidden, cfg.heads, cfg.ffn, causal=cfg.causal, seed=base + 1 + i))
    specs.append(LayerSpec(LayerNorm, cfg.hidden))
    nxt = base + cfg.layers + 2
    if cfg.mlm:
        specs.append(LayerSpec(MLMTransform, cfg.hidden, seed=nxt))
        nxt += 1
    specs.append(LayerSpec(Linear, cfg.hidden, cfg.vocab, bias=False, pad_to=cfg.vocab_pad, seed=nxt))
    return specs


MASK_TOKEN_ID = 103      # [MASK] in the BERT vocabulary


def mlm_mask(tokens, generator, vocab, mask_id=MASK_TOKEN_ID, ignore_index=-100):
    """BERT masking of a batch of token ids: 15 % of the positions of each sequence are chosen;
    the label is the original token there and ``ignore_index`` elsewhere; of the chosen inputs
    80 % become ``mask_id``, 10 % a random token, 10 % stay.  Returns (inputs, labels)."""
    B, S = tokens.shape
    n = max(1, int(round(0.15 * S)))
    order = torch.rand(B, S, generator=generator).argsort(dim=1)[:, :n]          # n distinct positions per row
    chosen = torch.zeros(B, S, dtype=torch.bool).scatter_(1, order, True)
    labels = torch.where(chosen, tokens, torch.full_like(tokens, ignore_index))
    roll = torch.rand(B, S, generator=generator)
    rand_tok = torch.randint(0, vocab, (B, S), generator=generator)
    inputs = tokens.clone()
    inputs[chosen & (roll < 0.8)] = mask_id
    swap = chosen & (roll >= 0.8) & (roll < 0.9)
    inputs[swap] = rand_tok[swap]
    return inputs, labels


def transformer_loss(cfg: TransformerConfig, ignore_index=-100):
    return CrossEntropyLoss(cfg.vocab, ignore_index)
