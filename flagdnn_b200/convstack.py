"""The ResNet-50 forward convolution stack as a workload for the conv path.

53 convolutions (v1.5: the stride of a down-sampling bottleneck sits on its
3x3): a 7x7 stride-2 stem, then [3, 4, 6, 3] bottlenecks of 1x1 / 3x3 / 1x1 at
widths 64 / 128 / 256 / 512 with 4x expansion, and a projection 1x1 on the
shortcut of each stage's first block.  Every convolution carries a BN-folded
per-channel scale and bias; all but each block's third 1x1 and the projection
are followed by ReLU (those two feed the residual add).

The convolutions and the pooling after the stem run through this library; the
residual add + ReLU is fused into each block's last convolution on request,
otherwise plain torch glue.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import conv_host, pool_host


@dataclass(frozen=True)
class ConvLayer:
    name: str
    cin: int
    cout: int
    k: int
    stride: int
    pad: int
    relu: bool
    hw_in: int            # input height = width

    @property
    def hw_out(self) -> int:
        return (self.hw_in + 2 * self.pad - self.k) // self.stride + 1

    def flops(self, batch: int) -> float:
        return 2.0 * batch * self.hw_out ** 2 * self.cout * self.cin * self.k ** 2

    def bytes(self, batch: int, itemsize: int = 2) -> float:
        return itemsize * (batch * self.cin * self.hw_in ** 2 + self.cout * self.cin * self.k ** 2
                           + 2 * self.cout + batch * self.cout * self.hw_out ** 2)

    @property
    def shape_key(self) -> Tuple[int, ...]:
        return (self.cin, self.hw_in, self.cout, self.k, self.stride, self.pad, int(self.relu))


def resnet50_conv_layers(image: int = 224) -> List[ConvLayer]:
    layers = [ConvLayer("stem", 3, 64, 7, 2, 3, True, image)]
    hw = layers[0].hw_out
    hw = (hw + 2 - 3) // 2 + 1  # 3x3 stride-2 max pool, padding 1
    cin = 64
    for stage, (blocks, width) in enumerate(zip((3, 4, 6, 3), (64, 128, 256, 512)), start=1):
        for block in range(blocks):
            stride = 2 if (block == 0 and stage > 1) else 1
            tag = f"s{stage}b{block}"
            layers.append(ConvLayer(f"{tag}.conv1", cin, width, 1, 1, 0, True, hw))
            layers.append(ConvLayer(f"{tag}.conv2", width, width, 3, stride, 1, True, hw))
            hw_out = layers[-1].hw_out
            layers.append(ConvLayer(f"{tag}.conv3", width, width * 4, 1, 1, 0, False, hw_out))
            if block == 0:
                layers.append(ConvLayer(f"{tag}.proj", cin, width * 4, 1, stride, 0, False, hw))
            cin = width * 4
            hw = hw_out
    return layers


def stack_totals(layers: List[ConvLayer], batch: int) -> Dict[str, float]:
    return {"flops": sum(l.flops(batch) for l in layers), "bytes": sum(l.bytes(batch) for l in layers),
            "convs": len(layers), "unique_shapes": len({l.shape_key for l in layers})}


def make_layer_params(layer: ConvLayer, seed: int, device, dtype=torch.bfloat16):
    """Random-init weight ~ N(0, 1/fan_in) (channels-last), scale ~ U(0.5, 1.5), bias ~ N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    fan_in = layer.cin * layer.k * layer.k
    w = torch.randn(layer.cout, layer.cin, layer.k, layer.k, generator=g) * fan_in ** -0.5
    scale = torch.rand(layer.cout, generator=g) + 0.5
    bias = torch.randn(layer.cout, generator=g) * 0.1
    w = w.to(dtype).to(device).contiguous(memory_format=torch.channels_last)
    return w, scale.to(dtype).to(device), bias.to(dtype).to(device)


def run_layer(layer: ConvLayer, x: torch.Tensor, params, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One convolution with its folded scale and bias; with ``residual`` the block's shortcut add and
    the ReLU after it happen in the same kernel (the layer's own ``relu`` flag is then moot)."""
    w, scale, bias = params
    if residual is not None:
        return conv_host.conv2d_bias_act(x, w, bias, stride=layer.stride, padding=layer.pad, scale=scale,
                                         relu=True, residual=residual)
    return conv_host.fused_conv2d_bias_relu(x, w, bias, stride=layer.stride, padding=layer.pad, scale=scale,
                                            activation="relu" if layer.relu else "none")


class ResNet50ConvStack:
    """All 53 convolutions with their parameters; ``forward`` chains them with torch glue."""

    def __init__(self, device, dtype=torch.bfloat16, seed: int = 0, image: int = 224):
        self.layers = resnet50_conv_layers(image)
        self.params = [make_layer_params(l, seed + i, device, dtype) for i, l in enumerate(self.layers)]
        self.device, self.dtype = device, dtype

    def forward(self, x: torch.Tensor, conv=run_layer, collect: Optional[list] = None,
                fuse_residual: bool = False) -> torch.Tensor:
        """x: [N, 3, H, W] channels-last.  ``conv(layer, x, params)`` computes one convolution
        (the library by default; tests pass an oracle).  ``collect`` receives (layer, input, output).
        With ``fuse_residual`` each block's third convolution takes the shortcut as its residual
        (``conv(layer, x, params, residual=...)``), so only the max-pool is left to torch."""
        def step(index, inp, residual=None):
            layer, params = self.layers[index], self.params[index]
            out = conv(layer, inp, params) if residual is None else conv(layer, inp, params, residual=residual)
            if collect is not None:
                collect.append((layer, inp, out))
            return out

        y = step(0, x)
        y = pool_host.max_pool2d(y, 3, 2, 1) if y.is_cuda else torch.nn.functional.max_pool2d(y, 3, 2, 1)
        index = 1
        for blocks in (3, 4, 6, 3):
            for block in range(blocks):
                identity = y
                t = step(index, y)
                t = step(index + 1, t)
                if block == 0:
                    identity = step(index + 3, y)          # projection shortcut
                if fuse_residual:
                    y = step(index + 2, t, residual=identity)
                else:
                    y = torch.relu(step(index + 2, t) + identity)
                index += 4 if block == 0 else 3
        return y
