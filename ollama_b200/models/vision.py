"""Image input for gemma3: the SigLIP vision tower and the multimodal projector that turn an image into rows of the text
model's embedding space.

The tensors are the ``v.*`` / ``mm.*`` entries of a multimodal GGUF (convert/convert_gemma3.go:155-188 names them: patch
embedding, position embedding, ``v.blk.N.{layer_norm1, attn_q, attn_k, attn_v, attn_output, layer_norm2, mlp.fc1, mlp.fc2}``,
``v.post_layernorm``, ``mm.mm_soft_emb_norm``, ``mm.mm_input_projection``), the hyper-parameters the ``gemma3.vision.*`` keys
(convert/convert_gemma3.go:134-147).  An image is resized to ``image_size`` squared (bilinear), scaled to [-1, 1], cut into
``patch_size`` squared patches; the tower is a pre-LayerNorm transformer encoder with full attention; the projector
average-pools the patch grid down to ``tokens_per_image`` positions, applies an RMSNorm and a linear map into the text width.
The reference hands the same work to its runner's image projector (server/images.go:716-787 picks the projector layers,
server/prompt.go:23-133 places ``[img-N]`` markers); here it is a few hundred matrix products per image on the device the text
model runs on, outside the token loop.
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ..ops import reference as R


@dataclass
class VisionConfig:
    n_layers: int
    d_model: int
    d_ff: int
    n_heads: int
    image_size: int
    patch_size: int
    channels: int = 3
    eps: float = 1e-6
    tokens_per_image: int = 256
    text_width: int = 0


def vision_config_from_gguf(g) -> VisionConfig | None:
    """The vision hyper-parameters of an opened GGUF, or None when it carries no vision tower."""
    arch = g.architecture
    if not g.has("v.patch_embedding.weight") or f"{arch}.vision.block_count" not in g.kv:
        return None
    u = lambda k, d=0: int(g.kv.get(f"{arch}.{k}", d))                                  # noqa: E731
    return VisionConfig(n_layers=u("vision.block_count"), d_model=u("vision.embedding_length"), d_ff=u("vision.feed_forward_length"),
                        n_heads=u("vision.attention.head_count"), image_size=u("vision.image_size", 896), patch_size=u("vision.patch_size", 14),
                        channels=u("vision.num_channels", 3), eps=float(g.kv.get(f"{arch}.vision.attention.layer_norm_epsilon", 1e-6)),
                        tokens_per_image=u("mm.tokens_per_image", 256), text_width=u("embedding_length"))


def preprocess(data: bytes, size: int) -> torch.Tensor:
    """Encoded image bytes (PNG, JPEG, ...) -> float tensor [3, size, size] in [-1, 1]: RGB, bilinear resize, (x / 255 - 0.5) / 0.5."""
    from PIL import Image
    img = Image.open(io.BytesIO(data)).convert("RGB").resize((size, size), Image.BILINEAR)
    x = torch.frombuffer(bytearray(img.tobytes()), dtype=torch.uint8).view(size, size, 3).permute(2, 0, 1).float()
    return (x / 255.0 - 0.5) / 0.5


def load_tower(g, device="cpu") -> "VisionTower | None":
    """The vision tower of an opened GGUF on ``device``, or None when the file has none."""
    from .weights import load_tensor
    cfg = vision_config_from_gguf(g)
    if cfg is None:
        return None
    return VisionTower(cfg, {n: load_tensor(g, n) for n in g.tensors if n.startswith(("v.", "mm."))}, device)


class VisionTower:
    """SigLIP encoder + gemma3 projector over dequantised tensors (fp32 on CPU, bf16 matrices with fp32 accumulation are not
    worth it here: an image is encoded once per request)."""

    def __init__(self, cfg: VisionConfig, tensors, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w: dict[str, torch.Tensor] = {}
        for name in tensors:
            if name.startswith(("v.", "mm.")):
                t = tensors[name]
                self.w[name] = (t.dequant() if hasattr(t, "dequant") else t).float().to(self.device)

    def _lin(self, x: torch.Tensor, name: str) -> torch.Tensor:
        y = x @ self.w[name + ".weight"].t()
        b = self.w.get(name + ".bias")
        return y + b if b is not None else y

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x, (x.shape[-1],), self.w[name + ".weight"], self.w.get(name + ".bias"), self.cfg.eps)

    @torch.no_grad()
    def patches(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [3, S, S] -> encoder output [n_patches, d_model]."""
        c = self.cfg
        side = c.image_size // c.patch_size
        w = self.w["v.patch_embedding.weight"].reshape(c.d_model, c.channels, c.patch_size, c.patch_size)
        x = F.conv2d(pixels.to(self.device)[None], w, self.w.get("v.patch_embedding.bias"), stride=c.patch_size)      # [1, d, side, side]
        x = x.flatten(2).transpose(1, 2)[0] + self.w["v.position_embedding.weight"][: side * side]
        hd = c.d_model // c.n_heads
        for i in range(c.n_layers):
            p = f"v.blk.{i}."
            h = self._ln(x, p + "layer_norm1")
            q = self._lin(h, p + "attn_q").view(-1, c.n_heads, hd).transpose(0, 1)
            k = self._lin(h, p + "attn_k").view(-1, c.n_heads, hd).transpose(0, 1)
            v = self._lin(h, p + "attn_v").view(-1, c.n_heads, hd).transpose(0, 1)
            a = torch.softmax((q @ k.transpose(1, 2)) / math.sqrt(hd), -1) @ v                  # full attention over the patches
            x = x + self._lin(a.transpose(0, 1).reshape(-1, c.d_model), p + "attn_output")
            h = self._ln(x, p + "layer_norm2")
            x = x + self._lin(R.gelu_tanh(self._lin(h, p + "mlp.fc1")), p + "mlp.fc2")
        return self._ln(x, "v.post_layernorm")

    @torch.no_grad()
    def project(self, feats: torch.Tensor) -> torch.Tensor:
        """Encoder output [n_patches, d_model] -> [tokens_per_image, text width]: average pool over the patch grid, RMSNorm, linear."""
        c = self.cfg
        side = c.image_size // c.patch_size
        tps = max(1, int(math.isqrt(c.tokens_per_image)))
        kernel = max(1, side // tps)
        grid = feats.t().reshape(1, c.d_model, side, side)
        pooled = F.avg_pool2d(grid, kernel, kernel).flatten(2)[0].t()                           # [tokens, d_model]
        normed = R.rmsnorm(pooled, self.w["mm.mm_soft_emb_norm.weight"], c.eps)
        # the projection keeps the checkpoint's orientation, [vision width, text width], and multiplies from the right
        return normed @ self.w["mm.mm_input_projection.weight"]

    def encode(self, data: bytes) -> torch.Tensor:
        """Encoded image -> rows of the text model's embedding space, [tokens_per_image, text width] fp32."""
        return self.project(self.patches(preprocess(data, self.cfg.image_size)))
