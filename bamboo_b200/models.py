"""Layer lists of the benchmark model families (token-input GPT decoder, BERT-style MLM
encoder) for ``PipelineModule``.

The reference's example models (``DeepSpeedExamples/pipeline_parallelism/gpt2.py:20-154``,
``bert.py:20-150``) have no embedding or vocabulary head and train on random activations;
the benchmark configurations ask for token inputs, learned position embeddings, pre-LN
blocks and a cross-entropy loss, so the layer list is:

    TokenEmbedding, TransformerBlock x L, LayerNorm, Linear(hidden -> vocab, no bias)

Initialisation: N(0, 0.02) weights, zero biases, unit LayerNorm gains; layer ``i`` of the
list draws from ``torch.Generator().manual_seed(seed * 1000 + i)`` in parameter-definition
order, so a stage (or a shadow copy of it) built on any rank holds identical values.
"""
from dataclasses import dataclass

from .layers import CrossEntropyLoss, LayerNorm, Linear, TokenEmbedding, TransformerBlock
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

    @property
    def padded_vocab(self):
        return (self.vocab + self.vocab_pad - 1) // self.vocab_pad * self.vocab_pad

    def flops_per_token(self):
        """Training FLOPs per token, dense attention count: 3 * (L*(24h^2 + 4sh) + 2hV)."""
        h = self.hidden
        return 3 * (self.layers * (24 * h * h + 4 * self.seq * h) + 2 * h * self.vocab)


GPT_TOY = TransformerConfig(layers=4, hidden=256, heads=4, ffn=1024, seq=128, vocab=1024)
GPT2_MEDIUM = TransformerConfig(layers=24, hidden=1024, heads=16, ffn=4096, seq=1024, vocab=50257)
BERT_LARGE = TransformerConfig(layers=24, hidden=1024, heads=16, ffn=4096, seq=512, vocab=30522, causal=False)
GPT_6_7B = TransformerConfig(layers=32, hidden=4096, heads=32, ffn=16384, seq=2048, vocab=50257)


def transformer_layer_specs(cfg: TransformerConfig, seed: int = 0):
    base = seed * 1000
    specs = [LayerSpec(TokenEmbedding, cfg.vocab, cfg.hidden, cfg.seq, seed=base)]
    for i in range(cfg.layers):
        specs.append(LayerSpec(TransformerBlock, cfg.hidden, cfg.heads, cfg.ffn, causal=cfg.causal, seed=base + 1 + i))
    specs.append(LayerSpec(LayerNorm, cfg.hidden))
    specs.append(LayerSpec(Linear, cfg.hidden, cfg.vocab, bias=False, pad_to=cfg.vocab_pad, seed=base + cfg.layers + 2))
    return specs


def transformer_loss(cfg: TransformerConfig, ignore_index=-100):
    return CrossEntropyLoss(cfg.vocab, ignore_index)
