"""Seeded synthetic GGUF weights and activations with the value distributions the benchmark
configurations state, generated directly on the GPU (no dataset or checkpoint is available):

  Q8_0: fp16 d = |N(0,1)|*0.02, int8 quants uniform in [-127, 127]
  Q4_0: fp16 d = |N(0,1)|*0.02, nibbles uniform
  Q4_K: fp16 d, dmin = |N(0,1)|*0.01, 12 scale bytes and 128 quant bytes uniform
  Q6_K: ql / qh uniform bytes, int8 sub-scales uniform in [-64, 63], fp16 d = |N(0,1)|*0.005

Scale fields are drawn as fp16 numbers and then viewed as bytes (random bytes would contain
NaN / Inf patterns).
"""

from __future__ import annotations

import torch

from .formats import Q4_0, Q4_K, Q6_K, Q8_0, get_format


def _half_bytes(shape, std, gen, device):
    vals = (torch.randn(shape, generator=gen, device=device).abs() * std).to(torch.float16)
    return vals.view(torch.uint8).reshape(*shape, 2)


def make_weights(encoding, n: int, k: int, seed: int, device) -> torch.Tensor:
    """Raw bytes (uint8, flat) of a random ``[n, k]`` weight."""
    fmt = get_format(encoding)
    nb = k // fmt.weights
    if k % fmt.weights:
        raise ValueError("K must be a multiple of the block size")
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    b = torch.randint(0, 256, (n, nb, fmt.nbytes), generator=gen, device=device, dtype=torch.uint8)
    if fmt is Q8_0:
        b[..., 0:2] = _half_bytes((n, nb), 0.02, gen, device)
        q = torch.randint(-127, 128, (n, nb, 32), generator=gen, device=device, dtype=torch.int8)
        b[..., 2:34] = q.view(torch.uint8)
    elif fmt is Q4_0:
        b[..., 0:2] = _half_bytes((n, nb), 0.02, gen, device)
    elif fmt is Q4_K:
        b[..., 0:2] = _half_bytes((n, nb), 0.01, gen, device)
        b[..., 2:4] = _half_bytes((n, nb), 0.01, gen, device)
    elif fmt is Q6_K:
        sc = torch.randint(-64, 64, (n, nb, 16), generator=gen, device=device, dtype=torch.int8)
        b[..., 192:208] = sc.view(torch.uint8)
        b[..., 208:210] = _half_bytes((n, nb), 0.005, gen, device)
    return b.reshape(-1)


def make_activations(m: int, k: int, seed: int, device, dtype=torch.bfloat16) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return torch.randn((m, k), generator=gen, device=device).to(dtype)
