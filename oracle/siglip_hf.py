"""Hugging Face eager SigLIP vision tower as the checker (test infrastructure, never the product path).

The reference validates its SigLIP megakernel against ``AutoModel(...).vision_model`` outputs
(reference ``src/ittai/siglip/kernel.py:675,701-702``) and runs the MAP pooling head through the torch
modules themselves (``:626-629``).  Built offline from the ViT-B/16 224-pixel config with seeded random init.
"""
from __future__ import annotations

import os
import time

import torch


def build_hf(seed: int = 2, dtype=torch.bfloat16, device="cpu", n_layers: int = 12):
    """Random-init ``SiglipVisionModel``: 12 layers, width 768, 12 heads, MLP 3072 GELU-tanh, LayerNorm eps 1e-6,
    196 patches + learned positions, MAP attention-pooling head.  ``.vision_model`` is what the reference's wrapper keeps."""
    from transformers import SiglipVisionConfig, SiglipVisionModel

    cfg = SiglipVisionConfig(hidden_size=768, intermediate_size=3072, num_hidden_layers=n_layers, num_attention_heads=12,
                             image_size=224, patch_size=16, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    torch.manual_seed(seed)
    model = SiglipVisionModel(cfg).to(dtype).eval()
    return model.to(device) if device != "cpu" else model


def pixels(batch: int, seed: int = 3) -> torch.Tensor:
    """fp32 [B, 3, 224, 224] drawn from N(0, 1) with a seeded CPU generator."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(batch, 3, 224, 224, generator=g)


@torch.no_grad()
def time_cpu(batch: int, iters: int = 3, threads: int | None = None):
    """Images per second of the eager bf16 tower on host cores."""
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    m = build_hf()
    px = pixels(batch).to(torch.bfloat16)
    m(pixel_values=px)
    t0 = time.perf_counter()
    for _ in range(iters):
        m(pixel_values=px)
    dt = (time.perf_counter() - t0) / iters
    return dict(img_s=batch / dt, ms=dt * 1e3, threads=threads, batch=batch)


def build_hf_naflex(seed: int = 2, dtype=torch.bfloat16, device="cpu", n_layers: int = 12, num_patches: int = 256):
    """Random-init ``Siglip2VisionModel`` at the base geometry: the variable-resolution (NaFlex) tower the reference's
    wrapper loads by default (``src/ittai/siglip/kernel.py:672``): Linear patch embedding over 16 x 16 x 3 patch rows, a
    16 x 16 learned position grid resized per image, key masks in every attention."""
    from transformers import Siglip2VisionConfig, Siglip2VisionModel

    cfg = Siglip2VisionConfig(hidden_size=768, intermediate_size=3072, num_hidden_layers=n_layers, num_attention_heads=12,
                              num_patches=num_patches, patch_size=16, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    torch.manual_seed(seed)
    model = Siglip2VisionModel(cfg).to(dtype).eval()
    return model.to(device) if device != "cpu" else model


def naflex_inputs(shapes, num_patches: int = 256, seed: int = 3):
    """Patch rows of images with the given (height, width) patch grids: N(0, 1) values for the valid rows, zeros after."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    B = len(shapes)
    px = torch.zeros(B, num_patches, 3 * 16 * 16)
    mask = torch.zeros(B, num_patches, dtype=torch.int64)
    for b, (h, w) in enumerate(shapes):
        px[b, :h * w] = torch.randn(h * w, 3 * 16 * 16, generator=g)
        mask[b, :h * w] = 1
    return {"pixel_values": px, "pixel_attention_mask": mask, "spatial_shapes": torch.tensor(shapes, dtype=torch.int64)}


def build_hf_so400m(naflex: bool = False, n_layers: int = 27, device="cpu", dtype=torch.bfloat16, seed: int = 5):
    """Random-init tower with the so400m widths (1152 wide, 16 heads of 72, MLP 4304): ``siglip2-so400m-patch14-384`` is
    the reference benchmark's default model (reference ``benchmarks/siglip.py:7``); ``naflex`` gives the same widths as a
    variable-resolution tower (patch 16, 256 patches)."""
    from transformers import Siglip2VisionConfig, Siglip2VisionModel, SiglipVisionConfig, SiglipVisionModel
    kw = dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=n_layers, num_attention_heads=16,
              hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    torch.manual_seed(seed)
    m = (Siglip2VisionModel(Siglip2VisionConfig(num_patches=256, patch_size=16, **kw)) if naflex else
         SiglipVisionModel(SiglipVisionConfig(image_size=384, patch_size=14, **kw)))
    return m.to(dtype).eval().to(device)
