"""``cast_model`` + forward + backward + one ``FlashAdamW`` step on third-party
architectures (the smoke test of the reference's ``test/test_thirdparty.py:271-283``).

The reference downloads configurations; here every model is a two-layer,
32-wide random-init instance built from its Hugging Face config class, so the
test needs no network and runs on CPU in well under a second per model.
"""

import warnings

import pytest
import torch

from flashoptim_b200 import FlashAdamW, FlashLion, cast_model

transformers = pytest.importorskip("transformers")

pytestmark = pytest.mark.thirdparty

_IDS = torch.randint(0, 100, (2, 16), generator=torch.Generator().manual_seed(0))
_TINY = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
             max_position_embeddings=32)


def _lm(batch=None):
    return dict(input_ids=_IDS, labels=_IDS), (lambda out: out.loss)


def _pooled(inputs):
    return inputs, (lambda out: out.pooler_output.float().pow(2).mean())


def _gpt2(t):
    return t.GPT2LMHeadModel(t.GPT2Config(vocab_size=128, n_embd=32, n_layer=2, n_head=4, n_positions=32)), *_lm()


def _bert(t):
    return t.BertForMaskedLM(t.BertConfig(**_TINY)), *_lm()


def _llama(t):
    return t.LlamaForCausalLM(t.LlamaConfig(**_TINY, num_key_value_heads=2)), *_lm()


def _qwen2(t):
    return t.Qwen2ForCausalLM(t.Qwen2Config(**_TINY, num_key_value_heads=2)), *_lm()


def _qwen3_moe(t):
    cfg = t.Qwen3MoeConfig(**_TINY, num_key_value_heads=2, num_experts=4, num_experts_per_tok=2,
                           moe_intermediate_size=32, head_dim=8)
    return t.Qwen3MoeForCausalLM(cfg), *_lm()


def _gemma2(t):
    return t.Gemma2ForCausalLM(t.Gemma2Config(**_TINY, num_key_value_heads=2, head_dim=8)), *_lm()


def _mamba(t):
    return t.MambaForCausalLM(t.MambaConfig(vocab_size=128, hidden_size=32, num_hidden_layers=2, state_size=8)), *_lm()


def _vit(t):
    cfg = t.ViTConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                      image_size=32, patch_size=8, num_labels=5)
    inputs = dict(pixel_values=torch.randn(2, 3, 32, 32).bfloat16(), labels=torch.tensor([1, 2]))
    return t.ViTForImageClassification(cfg), inputs, (lambda out: out.loss)


def _dinov2(t):
    cfg = t.Dinov2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    return t.Dinov2Model(cfg), *_pooled(dict(pixel_values=torch.randn(2, 3, 28, 28).bfloat16()))


def _clip_text(t):
    return t.CLIPTextModel(t.CLIPTextConfig(**_TINY)), *_pooled(dict(input_ids=_IDS))


def _whisper(t):
    cfg = t.WhisperConfig(vocab_size=128, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                          decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, num_mel_bins=16,
                          max_source_positions=16, max_target_positions=32, pad_token_id=0, bos_token_id=1,
                          eos_token_id=2, decoder_start_token_id=1)
    inputs = dict(input_features=torch.randn(2, 16, 32).bfloat16(), labels=_IDS)
    return t.WhisperForConditionalGeneration(cfg), inputs, (lambda out: out.loss)


_BUILDERS = {
    "gpt2": _gpt2, "bert": _bert, "llama": _llama, "qwen2": _qwen2, "qwen3_moe": _qwen3_moe, "gemma2": _gemma2,
    "mamba": _mamba, "vit": _vit, "dinov2": _dinov2, "clip_text": _clip_text, "whisper": _whisper,
}


@pytest.mark.parametrize("name", sorted(_BUILDERS))
@pytest.mark.parametrize("optimizer", [FlashAdamW, FlashLion])
def test_cast_forward_backward_step(name, optimizer):
    torch.manual_seed(0)
    try:
        model, inputs, loss_of = _BUILDERS[name](transformers)
    except (AttributeError, TypeError) as e:  # architecture or config argument not in this transformers version
        pytest.skip(f"{name}: {e}")
    shapes = {n: tuple(p.shape) for n, p in model.named_parameters()}
    tied_before = len({id(p) for p in model.parameters()})
    cast_model(model, torch.bfloat16)
    assert {n: tuple(p.shape) for n, p in model.named_parameters()} == shapes
    assert len({id(p) for p in model.parameters()}) == tied_before
    assert all(p.dtype == torch.bfloat16 for p in model.parameters())
    opt = optimizer(model.parameters(), lr=1e-3)
    before = [p.detach().clone() for p in model.parameters()]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        loss = loss_of(model(**inputs))
    assert torch.isfinite(loss)
    loss.backward()
    opt.step()
    opt.zero_grad()
    changed = sum(int(not torch.equal(a, b)) for a, b in zip(before, model.parameters()))
    assert changed >= len(before) // 2
    assert all(torch.isfinite(p).all() for p in model.parameters())
    # the optimizer state survives a save / load cycle on these parameter lists too
    opt2 = optimizer(model.parameters(), lr=1e-3)
    opt2.load_state_dict(opt.state_dict())
    assert len(opt2.state) == len(opt.state)
