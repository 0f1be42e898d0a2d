"""``cast_model`` + forward + backward + one ``FlashAdamW`` step on third-party
architectures (the smoke test of the reference's ``test/test_thirdparty.py:271-283``).

The reference downloads configurations; here every model is a two-layer,
32-wide random-init instance built from its Hugging Face config class, so the
test needs no network and runs on CPU in well under a second per model (ten of them once
more on the GPU, where the CUDA kernels meet these parameter lists).
timm, diffusers and open_clip are not installable offline: torchvision's ResNet
(batch norm, integer buffers), a Swin (integer ``relative_position_index``), a
small MLP-Mixer and a two-tower CLIP stand in for the reference's timm and
open_clip entries (``test/test_thirdparty.py:122-145``, ``:324-366``); its
diffusers UNet has no stand-in.
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


def _square(out):
    return out.float().pow(2).mean()


def _resnet(t):
    """Stands in for timm's resnet50 (``test/test_thirdparty.py:126``): BatchNorm layers, which
    ``cast_model`` keeps in fp32, and their integer ``num_batches_tracked`` buffers."""
    tv = pytest.importorskip("torchvision")
    return tv.models.resnet18(num_classes=10), dict(x=torch.randn(2, 3, 64, 64).bfloat16()), _square


def _swin(t):
    """timm's swin_tiny (``:128``): an integer ``relative_position_index`` buffer per block."""
    cfg = t.SwinConfig(image_size=32, patch_size=4, embed_dim=16, depths=[2, 2], num_heads=[2, 4], window_size=4,
                       num_labels=5)
    inputs = dict(pixel_values=torch.randn(2, 3, 32, 32).bfloat16(), labels=torch.tensor([1, 2]))
    return t.SwinForImageClassification(cfg), inputs, (lambda out: out.loss)


class _Mixer(torch.nn.Module):
    """timm's mixer_b16 (``:129``) in miniature: token- and channel-mixing MLPs, no conv, no attention."""

    def __init__(self, patches=16, dim=32, depth=2, classes=10):
        super().__init__()
        nn = torch.nn
        self.embed = nn.Linear(3 * 8 * 8, dim)
        self.blocks = nn.ModuleList(nn.ModuleDict(dict(
            n1=nn.LayerNorm(dim), tok=nn.Sequential(nn.Linear(patches, 2 * patches), nn.GELU(), nn.Linear(2 * patches, patches)),
            n2=nn.LayerNorm(dim), ch=nn.Sequential(nn.Linear(dim, 2 * dim), nn.GELU(), nn.Linear(2 * dim, dim)),
        )) for _ in range(depth))
        self.head = nn.Linear(dim, classes)

    def forward(self, x):
        b = x.shape[0]
        x = x.unfold(2, 8, 8).unfold(3, 8, 8).permute(0, 2, 3, 1, 4, 5).reshape(b, 16, -1)
        x = self.embed(x)
        for blk in self.blocks:
            x = x + blk["tok"](blk["n1"](x).transpose(1, 2)).transpose(1, 2)
            x = x + blk["ch"](blk["n2"](x))
        return self.head(x.mean(1))


def _mixer(t):
    return _Mixer(), dict(x=torch.randn(2, 3, 32, 32).bfloat16()), _square


def _clip_dual(t):
    """Stands in for open_clip's ViT-B-32 (``:324-366``): an image and a text tower with a shared loss."""
    cfg = t.CLIPConfig(
        text_config=dict(**_TINY, projection_dim=16),
        vision_config=dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                           image_size=32, patch_size=8, projection_dim=16),
        projection_dim=16)
    inputs = dict(input_ids=_IDS, pixel_values=torch.randn(2, 3, 32, 32).bfloat16(), return_loss=True)
    return t.CLIPModel(cfg), inputs, (lambda out: out.loss)


def _sam(t):
    cfg = t.SamConfig(
        vision_config=dict(hidden_size=32, output_channels=16, num_hidden_layers=2, num_attention_heads=4, image_size=64,
                           patch_size=16, window_size=2, global_attn_indexes=[1], mlp_dim=64, num_pos_feats=8),
        prompt_encoder_config=dict(hidden_size=16, image_size=64, patch_size=16, mask_input_channels=4),
        mask_decoder_config=dict(hidden_size=16, mlp_dim=32, num_hidden_layers=1, num_attention_heads=2,
                                 iou_head_hidden_dim=16))
    inputs = dict(pixel_values=torch.randn(1, 3, 64, 64).bfloat16(),
                  input_points=torch.tensor([[[[20.0, 20.0]]]]).bfloat16(), input_labels=torch.tensor([[[1]]]))
    return t.SamModel(cfg), inputs, (lambda out: out.pred_masks.float().pow(2).mean() + out.iou_scores.float().sum())


def _qwen35(t):
    cfg = t.Qwen3_5Config(text_config=dict(**_TINY, num_key_value_heads=2, head_dim=8, linear_num_value_heads=4,
                                           linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8))
    inputs, loss_of = _lm()
    # two layers are both linear-attention layers: no key/value cache to ask for a length
    return t.Qwen3_5ForCausalLM(cfg.text_config if hasattr(cfg, "text_config") else cfg), dict(inputs, use_cache=False), loss_of


_BUILDERS = {
    "gpt2": _gpt2, "bert": _bert, "llama": _llama, "qwen2": _qwen2, "qwen3_moe": _qwen3_moe, "gemma2": _gemma2,
    "mamba": _mamba, "vit": _vit, "dinov2": _dinov2, "clip_text": _clip_text, "whisper": _whisper,
    "resnet": _resnet, "swin": _swin, "mixer": _mixer, "clip_dual": _clip_dual, "sam": _sam, "qwen3_5": _qwen35,
}


# the architectures that have also been run through the CUDA kernels on a B200 (FlashAdamW); the
# others have only been run on CPU
_GPU_NAMES = ["bert", "clip_dual", "clip_text", "dinov2", "gemma2", "gpt2", "llama", "mamba", "mixer", "qwen2"]
_CASES = [(n, o, "cpu") for o in (FlashAdamW, FlashLion) for n in sorted(_BUILDERS)]
_CASES += [pytest.param(n, FlashAdamW, "cuda", marks=pytest.mark.gpu) for n in _GPU_NAMES]


@pytest.mark.parametrize("name,optimizer,device", _CASES)
def test_cast_forward_backward_step(name, optimizer, device):
    torch.manual_seed(0)
    try:
        model, inputs, loss_of = _BUILDERS[name](transformers)
    except (AttributeError, TypeError, ValueError) as e:  # architecture or config argument not in this transformers version
        pytest.skip(f"{name}: {e}")
    model = model.to(device)
    inputs = {k: v.to(device) if torch.is_tensor(v) else v for k, v in inputs.items()}
    shapes = {n: tuple(p.shape) for n, p in model.named_parameters()}
    tied_before = len({id(p) for p in model.parameters()})
    int_buffers = {n: b.dtype for n, b in model.named_buffers() if not b.dtype.is_floating_point}
    batch_norms = {id(p) for m in model.modules() if isinstance(m, torch.nn.modules.batchnorm._BatchNorm)
                   for p in m.parameters()}
    cast_model(model, torch.bfloat16)
    assert {n: tuple(p.shape) for n, p in model.named_parameters()} == shapes
    assert len({id(p) for p in model.parameters()}) == tied_before
    # everything narrow except batch-norm parameters, which stay fp32; integer buffers untouched
    assert all(p.dtype == (torch.float32 if id(p) in batch_norms else torch.bfloat16) for p in model.parameters())
    assert {n: b.dtype for n, b in model.named_buffers() if not b.dtype.is_floating_point} == int_buffers
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
