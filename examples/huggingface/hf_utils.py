"""Helpers for the Hugging Face examples: a registry of model families, synthetic inputs, size and FLOP counts.

Covers the families of the reference's examples/huggingface/pippy_*.py (bert, blenderbot, camemBert, convBert,
deberta, debertaV2, distilBert, electra, fnet, gpt2, gptNeo, layoutLM, mbart, megatronBert, mobileBert, opt,
trOCR, xlnet) plus llama, and the input builders of examples/huggingface/hf_utils.py:71-225.  Models are
random-initialised from a config (there is no network): `size="tiny"` gives a 4-layer, 64-wide model for CPU
tests, `size="base"` the family's default config.  Nothing is installed at import time.
"""
from dataclasses import dataclass, field
from typing import Callable, Dict, Tuple

import torch


@dataclass
class Family:
    """One model family: how to build it, where its layers live and what it takes as input."""

    config_cls: str
    model_cls: str
    layer_path: str                       # dotted path of the ModuleList that is cut into stages
    tiny: dict                            # config overrides of the small test model
    inputs: str = "ids"                   # ids | ids_bbox | seq2seq
    n_layers: Callable = field(default=lambda cfg: cfg.num_hidden_layers)


_ENC = dict(num_hidden_layers=4, hidden_size=64, num_attention_heads=4, intermediate_size=128,
            vocab_size=128, max_position_embeddings=64)
_S2S = dict(encoder_layers=2, decoder_layers=4, d_model=64, encoder_attention_heads=4, decoder_attention_heads=4,
            encoder_ffn_dim=128, decoder_ffn_dim=128, vocab_size=128, max_position_embeddings=64)

FAMILIES: Dict[str, Family] = {
    "bert": Family("BertConfig", "BertForMaskedLM", "bert.encoder.layer", _ENC),
    "camembert": Family("CamembertConfig", "CamembertForMaskedLM", "roberta.encoder.layer", _ENC),
    "convbert": Family("ConvBertConfig", "ConvBertForMaskedLM", "convbert.encoder.layer",
                       dict(_ENC, embedding_size=64)),
    "deberta": Family("DebertaConfig", "DebertaForMaskedLM", "deberta.encoder.layer", _ENC),
    "debertav2": Family("DebertaV2Config", "DebertaV2ForMaskedLM", "deberta.encoder.layer", _ENC),
    "distilbert": Family("DistilBertConfig", "DistilBertForMaskedLM", "distilbert.transformer.layer",
                         dict(n_layers=4, dim=64, n_heads=4, hidden_dim=128, vocab_size=128,
                              max_position_embeddings=64), n_layers=lambda c: c.n_layers),
    "electra": Family("ElectraConfig", "ElectraForMaskedLM", "electra.encoder.layer",
                      dict(_ENC, embedding_size=64)),
    "fnet": Family("FNetConfig", "FNetForMaskedLM", "fnet.encoder.layer",
                   dict(num_hidden_layers=4, hidden_size=64, intermediate_size=128, vocab_size=128,
                        max_position_embeddings=64)),
    "gpt2": Family("GPT2Config", "GPT2LMHeadModel", "transformer.h",
                   dict(n_layer=4, n_embd=64, n_head=4, vocab_size=128, n_positions=64),
                   n_layers=lambda c: c.n_layer),
    "gptneo": Family("GPTNeoConfig", "GPTNeoForCausalLM", "transformer.h",
                     dict(num_layers=4, hidden_size=64, num_heads=4, vocab_size=128, max_position_embeddings=64,
                          attention_types=[[["global", "local"], 2]], window_size=8),
                     n_layers=lambda c: c.num_layers),
    "layoutlm": Family("LayoutLMConfig", "LayoutLMForMaskedLM", "layoutlm.encoder.layer", _ENC, inputs="ids_bbox"),
    "llama": Family("LlamaConfig", "LlamaForCausalLM", "model.layers",
                    dict(num_hidden_layers=4, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                         intermediate_size=128, vocab_size=128, max_position_embeddings=64)),
    "mbart": Family("MBartConfig", "MBartForConditionalGeneration", "model.decoder.layers", _S2S, inputs="seq2seq",
                    n_layers=lambda c: c.decoder_layers),
    "blenderbot": Family("BlenderbotConfig", "BlenderbotForConditionalGeneration", "model.decoder.layers", _S2S,
                         inputs="seq2seq", n_layers=lambda c: c.decoder_layers),
    "megatronbert": Family("MegatronBertConfig", "MegatronBertForMaskedLM", "bert.encoder.layer", _ENC),
    "mobilebert": Family("MobileBertConfig", "MobileBertForMaskedLM", "mobilebert.encoder.layer",
                         dict(_ENC, embedding_size=32, intra_bottleneck_size=32)),
    "opt": Family("OPTConfig", "OPTForCausalLM", "model.decoder.layers",
                  dict(num_hidden_layers=4, hidden_size=64, num_attention_heads=4, ffn_dim=128, vocab_size=128,
                       max_position_embeddings=64, word_embed_proj_dim=64)),
    "trocr": Family("TrOCRConfig", "TrOCRForCausalLM", "model.decoder.layers",
                    dict(decoder_layers=4, d_model=64, decoder_attention_heads=4, decoder_ffn_dim=128,
                         vocab_size=128, max_position_embeddings=64), n_layers=lambda c: c.decoder_layers),
    "xlnet": Family("XLNetConfig", "XLNetLMHeadModel", "transformer.layer",
                    dict(n_layer=4, d_model=64, n_head=4, d_inner=128, vocab_size=128),
                    n_layers=lambda c: c.n_layer),
}


def build_model(name: str, size: str = "tiny"):
    """Random-initialised model of family `name`; returns (model in eval mode, config, Family)."""
    import transformers

    fam = FAMILIES[name]
    overrides = dict(fam.tiny) if size == "tiny" else {}
    config = getattr(transformers, fam.config_cls)(**overrides)
    # Key/value caches are Python objects that cannot cross a stage boundary; XLNet's memories likewise.
    for attr in ("use_cache", "use_mems_eval", "use_mems_train"):
        if hasattr(config, attr):
            setattr(config, attr, False)
    model = getattr(transformers, fam.model_cls)(config)
    return model.eval(), config, fam


def generate_inputs(name: str, config, batch: int, seq_len: int = 16, device="cpu") -> Tuple[tuple, dict]:
    """Synthetic (args, kwargs) of the full batch for family `name` (reference hf_utils.py:71-225)."""
    fam = FAMILIES[name]
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(2, config.vocab_size, (batch, seq_len), generator=g).to(device)
    if fam.inputs == "ids":
        return (ids,), {}
    if fam.inputs == "ids_bbox":
        return (ids, torch.zeros(batch, seq_len, 4, dtype=torch.long, device=device)), {}
    if fam.inputs == "seq2seq":
        return (ids,), {"decoder_input_ids": ids.clone()}
    raise ValueError(fam.inputs)


def equal_layer_split(name: str, config, n_stages: int) -> dict:
    """split_spec that starts a stage at every (layers / n_stages)-th block (reference pippy_gpt2.py:58-66)."""
    from pippy_b200 import SplitPoint

    fam = FAMILIES[name]
    layers = fam.n_layers(config)
    if n_stages > layers:
        raise ValueError(f"{name}: {n_stages} stages but only {layers} layers")
    per = layers // n_stages
    return {f"{fam.layer_path}.{i * per}": SplitPoint.BEGINNING for i in range(1, n_stages)}


def get_number_of_params(model) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad)


def calc_flop(config, batch: int, seq_len: int, n_params: int) -> float:
    """Forward FLOPs of one batch: 2 per parameter per token plus the attention score/value products."""
    hidden = getattr(config, "hidden_size", None) or getattr(config, "d_model", None) or getattr(config, "n_embd", 0)
    layers = (getattr(config, "num_hidden_layers", None) or getattr(config, "n_layer", None)
              or getattr(config, "decoder_layers", 0))
    return 2.0 * n_params * batch * seq_len + 4.0 * layers * batch * seq_len * seq_len * hidden
