"""Synthetic parameter lists with the shapes of the benchmark configurations.

``unet_2p6b``: 70 transformer blocks at width 1280 (4x[1280,1280], [10240,1280], [1280,5120], 3 norm
weight+bias pairs), 20 blocks of the same recipe at width 640, and 36/24/12 3x3 convs at 1280/640/320
channels: 1152 tensors, 2 597 068 800 parameters.  ``dit_11b``: 100 blocks of width 3072 (qkv, out, two
MLP matrices, 2 norms): 600 tensors, 11 325 235 200 parameters.  Building parameters from a shape list
follows the reference's tuner (src/kaon/tune.py:69-75).
"""
from __future__ import annotations

import math


def _block(width: int) -> list[tuple[int, ...]]:
    w = width
    return [(w, w)] * 4 + [(8 * w, w), (w, 4 * w)] + [(w,)] * 6


def unet_2p6b() -> list[tuple[int, ...]]:
    shapes: list[tuple[int, ...]] = []
    for _ in range(70):
        shapes += _block(1280)
    for _ in range(20):
        shapes += _block(640)
    shapes += [(1280, 1280, 3, 3)] * 36 + [(640, 640, 3, 3)] * 24 + [(320, 320, 3, 3)] * 12
    return shapes


def dit_11b() -> list[tuple[int, ...]]:
    shapes: list[tuple[int, ...]] = []
    for _ in range(100):
        shapes += [(9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288), (3072,), (3072,)]
    return shapes


def dit_block() -> list[tuple[int, ...]]:
    """One width-3072 DiT block (113 M parameters)."""
    return [(9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288), (3072,), (3072,)]


def unet_sample() -> list[tuple[int, ...]]:
    """One width-1280 block plus one [1280,1280,3,3] conv: the bounded sample the CPU baseline times."""
    return _block(1280) + [(1280, 1280, 3, 3)]


def unet_mid() -> list[tuple[int, ...]]:
    """Eight width-1280 blocks plus four [1280,1280,3,3] convs (269 M parameters): more than ten times the
    L2 cache per step, yet small enough to hold a few GB on the device - the list profiler captures use."""
    shapes: list[tuple[int, ...]] = []
    for _ in range(8):
        shapes += _block(1280)
    return shapes + [(1280, 1280, 3, 3)] * 4


def unet_mid_odd() -> list[tuple[int, ...]]:
    """``unet_mid`` plus the odd tensors a real UNet has at its ends: a [320,4,3,3] input convolution (rows
    of 36 elements), a [4,320,3,3] output convolution, a [333,77] table - shapes that cannot take the
    streaming launches and must not take the rest of the list off them."""
    return unet_mid() + [(320, 4, 3, 3), (4, 320, 3, 3), (333, 77)]


def numel(shapes) -> int:
    return sum(math.prod(s) for s in shapes)


WORKLOADS = {"unet_2p6b": unet_2p6b, "dit_11b": dit_11b, "dit_block": dit_block, "unet_sample": unet_sample,
             "unet_mid": unet_mid, "unet_mid_odd": unet_mid_odd}
