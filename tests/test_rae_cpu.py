"""Representation autoencoder: SigLIP encoder and MAE decoder against the transformers classes, LPIPS against a
torchvision VGG-16 with the formula restated, the DINO discriminator's structure, and the GAN trainer."""
import math
import os
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

ENC = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=32, patch_size=8)
DEC = dict(decoder_hidden_size=48, decoder_num_hidden_layers=2, decoder_num_attention_heads=4, decoder_intermediate_size=96)


def _model(**kw):
    from lmms_engine_b200.mapping_func import create_model_from_config

    torch.manual_seed(0)
    return create_model_from_config("rae_siglip", dict(encoder_config=ENC, decoder_config=DEC, **kw))


def test_encoder_and_decoder_match_transformers():
    from transformers import SiglipVisionConfig, SiglipVisionModel, ViTMAEConfig
    from transformers.models.vit_mae.modeling_vit_mae import ViTMAEDecoder, get_2d_sincos_pos_embed

    model = _model(noise_tau=0.0).eval()
    hf_enc = SiglipVisionModel(SiglipVisionConfig(**ENC, attn_implementation="eager")).vision_model.eval()
    sd = {k: v for k, v in hf_enc.state_dict().items() if not k.startswith("head.") and not k.startswith("post_layernorm.")}
    missing, unexpected = model.encoder.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    x = torch.rand(2, 3, 32, 32)
    with torch.no_grad():
        hs = hf_enc(pixel_values=(x - 0.5) / 0.5).last_hidden_state  # its own post_layernorm is affine (ones / zeros at init)
        want = hs.transpose(1, 2).reshape(2, 32, 4, 4)
        got = model.encode(x)
    assert (got - want).abs().max() < 2e-5

    mae_cfg = ViTMAEConfig(hidden_size=32, patch_size=8, image_size=32, num_channels=3, layer_norm_eps=1e-12, **DEC, attn_implementation="eager")
    hf_dec = ViTMAEDecoder(mae_cfg, num_patches=16).eval()
    with torch.no_grad():
        for p in hf_dec.parameters():
            if p.requires_grad:
                p.normal_(0, 0.05)
    sd = {k: v for k, v in hf_dec.state_dict().items() if k not in ("mask_token", "decoder_pos_embed")}
    missing, unexpected = model.decoder.load_state_dict(sd, strict=False)
    assert set(missing) == {"trainable_cls_token", "decoder_pos_embed"} and not unexpected, (missing, unexpected)
    table = torch.from_numpy(get_2d_sincos_pos_embed(48, 4, add_cls_token=True)).float()
    assert (model.decoder.decoder_pos_embed[0] - table).abs().max() < 1e-6
    lat = torch.randn(2, 16, 32)
    with torch.no_grad():
        h = hf_dec.decoder_embed(lat)
        h = torch.cat([model.decoder.trainable_cls_token.expand(2, -1, -1), h], 1) + table
        for layer in hf_dec.decoder_layers:
            out = layer(h)
            h = out[0] if isinstance(out, tuple) else out
        want = hf_dec.decoder_pred(hf_dec.decoder_norm(h))[:, 1:]
        got, _ = model.decoder(lat)
    assert (got - want).abs().max() < 3e-5
    # un-patchify is the inverse of cutting an image into (row, column, pixel-row, pixel-column, channel) patches
    img = torch.rand(2, 3, 32, 32)
    patches = img.view(2, 3, 4, 8, 4, 8).permute(0, 2, 4, 3, 5, 1).reshape(2, 16, -1)
    assert torch.equal(model.decoder.unpatchify(patches), img)


def test_autoencoder_forward_noise_and_latent_normalisation():
    model = _model(noise_tau=0.5, latent_mean=[0.1], latent_var=[4.0])
    x = torch.rand(3, 3, 40, 40)  # resized to the encoder's input size
    model.eval()
    z = model.encode(x)
    assert z.shape == (3, 32, 4, 4) and torch.equal(z, model.encode(x))  # no noise in eval mode
    model.train()
    assert not torch.equal(model.encode(x), z)
    out = model(pixel_values=x)
    assert out["out_pixels"].shape == (3, 3, 32, 32) and out["loss"].requires_grad
    out["loss"].backward()
    assert all(p.grad is None for p in model.encoder.parameters())
    assert model.last_layer().grad.abs().sum() > 0
    # normalisation is undone by decode
    model.eval()
    plain = _model(noise_tau=0.5).eval()
    plain.load_state_dict(model.state_dict())
    with torch.no_grad():
        assert (plain.decode(plain.encode(x))["out_pixels"] - model.decode(model.encode(x))["out_pixels"]).abs().max() < 1e-4


def test_lpips_matches_restated_formula_on_torchvision_vgg(tmp_path):
    tv = pytest.importorskip("torchvision")
    from lmms_engine_b200.models.rae import Lpips

    torch.manual_seed(0)
    vgg = tv.models.vgg16(weights=None).eval()
    torch.save(vgg.state_dict(), tmp_path / "vgg16.pth")
    lins = {f"lin{i}.model.1.weight": torch.rand(1, c, 1, 1) for i, c in enumerate((64, 128, 256, 512, 512))}
    torch.save(lins, tmp_path / "lins.pth")
    with pytest.raises(FileNotFoundError):
        Lpips()
    lp = Lpips(str(tmp_path / "vgg16.pth"), str(tmp_path / "lins.pth"))
    assert not any(p.requires_grad for p in lp.parameters())
    a, b = torch.rand(2, 3, 64, 64) * 2 - 1, torch.rand(2, 3, 64, 64) * 2 - 1
    shift, scale = torch.tensor([-0.030, -0.088, -0.188]).view(1, 3, 1, 1), torch.tensor([0.458, 0.448, 0.450]).view(1, 3, 1, 1)

    def feats(x):
        out, h = [], (x - shift) / scale
        for i, layer in enumerate(vgg.features[:30]):
            h = layer(h)
            if i in (3, 8, 15, 22, 29):
                out.append(h / (h.pow(2).sum(1, keepdim=True).sqrt() + 1e-10))
        return out

    with torch.no_grad():
        want = sum((F.conv2d((fa - fb) ** 2, lins[f"lin{i}.model.1.weight"])).mean((2, 3)) for i, (fa, fb) in enumerate(zip(feats(a), feats(b))))
        got = lp(a, b, reduction="none")
    assert (got.flatten() - want.flatten()).abs().max() < 1e-5
    assert float(lp(a, a)) == 0.0
    a.requires_grad_(True)
    lp(a, b).backward()
    assert a.grad.abs().sum() > 0


def _dino_reference(sd, x, heads, key_depths):
    x = F.interpolate(x, size=(224, 224), mode="bilinear", align_corners=False)
    mean, std = torch.tensor((0.485, 0.456, 0.406)).view(1, 3, 1, 1), torch.tensor((0.229, 0.224, 0.225)).view(1, 3, 1, 1)
    x = x * (0.5 / std) + (0.5 - mean) / std
    h = F.conv2d(x, sd["patch_embed.proj.weight"], sd["patch_embed.proj.bias"], stride=sd["patch_embed.proj.weight"].shape[-1])
    h = h.flatten(2).transpose(1, 2)
    h = torch.cat([sd["cls_token"].expand(h.shape[0], -1, -1), h], 1) + sd["pos_embed"]
    D = h.shape[-1]
    acts, depth = [], len({k.split(".")[1] for k in sd if k.startswith("blocks.")})
    for i in range(depth):
        p = f"blocks.{i}."
        y = F.layer_norm(h, (D,), sd[p + "norm1.weight"], sd[p + "norm1.bias"], 1e-6)
        qkv = (y @ sd[p + "attn.qkv.weight"].T + sd[p + "attn.qkv.bias"]).view(h.shape[0], -1, 3, heads, D // heads).permute(2, 0, 3, 1, 4)
        att = (qkv[0] @ qkv[1].transpose(-1, -2) / math.sqrt(D // heads)).softmax(-1) @ qkv[2]
        h = h + att.transpose(1, 2).reshape(h.shape) @ sd[p + "attn.proj.weight"].T + sd[p + "attn.proj.bias"]
        y = F.layer_norm(h, (D,), sd[p + "norm2.weight"], sd[p + "norm2.bias"], 1e-6)
        y = F.gelu(y @ sd[p + "mlp.fc1.weight"].T + sd[p + "mlp.fc1.bias"], approximate="tanh")
        h = h + y @ sd[p + "mlp.fc2.weight"].T + sd[p + "mlp.fc2.bias"]
        if i in key_depths:
            acts.append(h[:, 1:].transpose(1, 2))
    return [h[:, 1:].transpose(1, 2)] + acts


def test_dino_discriminator_taps_a_frozen_backbone(tmp_path):
    from lmms_engine_b200.models.rae import DinoDiscriminator, FrozenDino

    torch.manual_seed(0)
    spec = dict(depth=3, patch_size=32, embed_dim=32, num_heads=4, mlp_ratio=2.0)
    src = FrozenDino(key_depths=(0, 2), **spec)
    with torch.no_grad():
        for p in src.parameters():
            p.normal_(0, 0.1)
    torch.save(src.state_dict(), tmp_path / "dino.pth")
    with pytest.raises(FileNotFoundError):
        DinoDiscriminator(backbone=spec)
    disc = DinoDiscriminator(str(tmp_path / "dino.pth"), ks=3, key_depths=(0, 2), backbone=spec)
    trainable = [n for n, p in disc.named_parameters() if p.requires_grad]
    assert trainable and all(n.startswith("heads.") for n in trainable)
    assert any("weight_orig" in n for n in trainable)  # spectral normalisation on the head convolutions
    disc.train()
    assert not disc.dino.training
    x = torch.rand(2, 3, 64, 64) * 2 - 1
    sd = {k: v.clone() for k, v in disc.dino.state_dict().items()}
    for k, v in sd.items():
        if k.endswith("attn.qkv.bias"):
            assert float(v[32:64].abs().sum()) == 0.0  # key bias zeroed at load
    with torch.no_grad():
        acts = disc.dino(x)
        want = _dino_reference(sd, x, 4, (0, 2))
    assert len(acts) == 3 and acts[0].shape == (2, 32, 49)
    for a, w in zip(acts, want):
        assert (a - w).abs().max() < 1e-4
    logits = disc(x)
    assert logits.shape == (2, 3 * 49)
    logits.mean().backward()
    assert all(p.grad is None for p in disc.dino.parameters())


def test_rae_trainer_runs_the_full_recipe(tmp_path):
    """L1 + LPIPS + adversarial generator steps and discriminator steps on random-weight critics."""
    from tests.test_trainers_cpu import _run, _tensors

    spec = {"pixel_values": {"shape": [3, 32, 32]}}
    gan = dict(allow_random_critics=True, backbone=dict(depth=2, patch_size=32, embed_dim=32, num_heads=4, mlp_ratio=2.0), key_depths=(0,),
               ks=3, discriminator_start_step=0, discriminator_loss_start_step=1, lpips_start_step=0)
    hist, runner = _run(tmp_path, "rae_trainer", "rae_siglip", dict(encoder_config=ENC, decoder_config=DEC), _tensors(spec),
                        per_device_train_batch_size=2, steps=3, gan_config=gan)
    tr = runner.trainer
    assert tr.ema_state and tr.lpips is not None and type(tr.discriminator).__name__ == "DinoDiscriminator"
    parts = tr.loss_parts
    assert parts["lpips_loss"] > 0 and parts["disc_loss"] > 0 and parts["gan_loss"] > 0 and parts["adaptive_weight"] > 0
    ck = tr.save_checkpoints(str(tmp_path / "out"))
    saved = torch.load(os.path.join(ck, "model.pt"))
    assert not any(k.startswith("discriminator") for k in saved)
    heads = torch.load(os.path.join(ck, "discriminator.pt"))["discriminator"]
    assert heads and not any(k.startswith("dino.") for k in heads)
    # without critic weights the trainer refuses instead of training on noise
    with pytest.raises(FileNotFoundError):
        _run(tmp_path, "rae_trainer", "rae_siglip", dict(encoder_config=ENC, decoder_config=DEC), _tensors(spec), per_device_train_batch_size=2, steps=1)


def test_adaptive_weight_from_the_last_layers_input_and_output_equals_the_weight_gradient():
    """``d_output^T @ input`` is the gradient with respect to the last layer's weight: the trainer's sharding-proof form of
    the GAN weight equals differentiating the parameter itself."""
    import types

    from lmms_engine_b200.mapping_func import create_model_from_config
    from lmms_engine_b200.train.fsdp2.extra_trainers import RaeTrainer

    torch.manual_seed(0)
    model = create_model_from_config("rae_siglip", dict(image_size=32, patch_size=8, encoder_dim=32, encoder_depth=1, encoder_heads=2,
                                                        decoder_dim=32, decoder_depth=1, decoder_heads=2)).train()
    x = torch.rand(2, 3, 32, 32)
    fake = types.SimpleNamespace(model=model, max_d_weight=1e4)
    rec = RaeTrainer.reconstruct(fake, x).float() if hasattr(RaeTrainer, "reconstruct") else model(pixel_values=x)["out_pixels"]
    rec_loss, g_loss = (rec - x).abs().mean(), (rec ** 2).mean() * 3.0
    assert model.last_layer_io() is not None
    got = RaeTrainer.adaptive_weight(fake, rec_loss, g_loss)
    last = model.last_layer()
    want = torch.autograd.grad(rec_loss, last, retain_graph=True)[0].norm() / (torch.autograd.grad(g_loss, last, retain_graph=True)[0].norm() + 1e-6)
    assert abs(float(got) - float(want)) < 1e-4 * float(want)
